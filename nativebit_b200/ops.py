"""Thin torch-tensor wrappers over the C ABI (device pointers in, device tensors out).

torch is used for device memory and streams only; all arithmetic happens in the kernels of
libnativebit_b200.so.  Every function requires CUDA tensors and raises otherwise.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import NB_BF16, NB_F16, NB_F32

_DTYPE = {torch.float32: NB_F32, torch.float16: NB_F16, torch.bfloat16: NB_BF16}


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """cudaStream_t of torch's current stream on the current device."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("nativebit_b200 runs on CUDA tensors only (no CPU fallback); got a "
                               f"{t.device} tensor")
        if not t.is_contiguous():
            raise RuntimeError("nativebit_b200 needs contiguous tensors")


def packed_nbytes(count: int, bits: int) -> int:
    """Bytes the reference's packers emit for `count` indices (nativebit/pack.py:21-41, 75-82, 97-116)."""
    return 3 * ((count + 7) // 8) if bits == 3 else (count * bits + 7) // 8


def unpack(packed: torch.Tensor, bits: int, count: int) -> torch.Tensor:
    """Packed bytes -> uint8 indices, one per byte (nativebit/pack.py:44-68, 85-90, 119-138)."""
    _need_cuda(packed)
    if packed.dtype != torch.uint8:
        raise RuntimeError("packed indices must be uint8")
    if packed.numel() < packed_nbytes(count, bits):
        raise RuntimeError(f"packed buffer too small: {packed.numel()} bytes for {count} {bits}-bit indices")
    out = torch.empty(count, dtype=torch.uint8, device=packed.device)
    with torch.cuda.device(packed.device):
        _lib.check(_lib.lib().nb_unpack(packed.data_ptr(), bits, count, out.data_ptr(), _stream()), "nb_unpack")
    return out


def pack(indices: torch.Tensor, bits: int) -> torch.Tensor:
    """uint8 indices -> packed bytes in the reference layout (nativebit/pack.py:21-41, 75-82, 97-116;
    inference/triton_kernel.py:199-220)."""
    _need_cuda(indices)
    if indices.dtype != torch.uint8:
        raise RuntimeError("indices must be uint8")
    flat = indices.reshape(-1)
    out = torch.empty(packed_nbytes(flat.numel(), bits), dtype=torch.uint8, device=indices.device)
    with torch.cuda.device(indices.device):
        _lib.check(_lib.lib().nb_pack(flat.data_ptr(), bits, flat.numel(), out.data_ptr(), _stream()), "nb_pack")
    return out


def dequant(packed: torch.Tensor, codebook: torch.Tensor, bits: int, block_size: int, shape,
            dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Whole-weight gather W[r, c] = codebook[b, idx[b, t]] (nativebit/pack.py:145-169)."""
    _need_cuda(packed, codebook)
    n_rows, n_cols = int(shape[0]), int(shape[1])
    total = n_rows * n_cols
    n_blocks = (total + block_size - 1) // block_size
    if codebook.dtype not in (torch.float16, torch.float32) or codebook.numel() != n_blocks * (1 << bits):
        raise RuntimeError(f"codebook must be fp16/fp32 with {n_blocks} x {1 << bits} entries")
    if packed.dtype != torch.uint8 or packed.numel() < packed_nbytes(n_blocks * block_size, bits):
        raise RuntimeError("packed buffer has the wrong dtype or is too small")
    out = torch.empty(n_rows, n_cols, dtype=dtype, device=packed.device)
    with torch.cuda.device(packed.device):
        _lib.check(_lib.lib().nb_dequant(packed.data_ptr(), codebook.data_ptr(), _DTYPE[codebook.dtype], bits, block_size,
                                         n_rows, n_cols, out.data_ptr(), _DTYPE[dtype], _stream()), "nb_dequant")
    return out


def quantize(weight: torch.Tensor, codebook: torch.Tensor, block_size: int) -> torch.Tensor:
    """Nearest-entry indices (num_blocks * block_size,) uint8 of a dense fp32 weight
    (nativebit/pack.py:176-199, inference/pack.py:21-35)."""
    _need_cuda(weight, codebook)
    if weight.dtype != torch.float32 or codebook.dtype not in (torch.float16, torch.float32):
        raise RuntimeError("quantize needs an fp32 weight and an fp16/fp32 codebook")
    total = weight.numel()
    nb, ne = codebook.shape
    if nb != (total + block_size - 1) // block_size:
        raise RuntimeError(f"codebook has {nb} blocks, the weight needs {(total + block_size - 1) // block_size}")
    out = torch.empty(nb * block_size, dtype=torch.uint8, device=weight.device)
    with torch.cuda.device(weight.device):
        _lib.check(_lib.lib().nb_quantize(weight.data_ptr(), total, codebook.data_ptr(), _DTYPE[codebook.dtype], ne, block_size,
                                          out.data_ptr(), _stream()), "nb_quantize")
    return out


_workspaces: dict = {}
_ws_need: dict = {}


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised scratch for split-K launches, one per (device, stream), grown on demand."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 4 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def workspace_status(ws: torch.Tensor) -> int:
    """The status word of a GEMV workspace (0, or NB_ERR_TIMEOUT = 6 if a bounded wait ran out); synchronises."""
    return int(ws[4095 * 4:4096 * 4].view(torch.int32).item())


def gemv_workspace_bytes(m: int, n: int, k: int, bits: int, block_size: int) -> int:
    key = (m, n, k, bits, block_size)
    need = _ws_need.get(key)
    if need is None:
        need = _ws_need[key] = int(_lib.lib().nb_gemv_workspace_bytes(m, n, k, bits, block_size))
        if need == 0:
            raise RuntimeError(f"nb_gemv does not support M={m} N={n} K={k} bits={bits} block_size={block_size} "
                               "(needs 1 <= M <= 16, bits in {2,3,4}, block_size 128, K % 128 == 0)")
    return need


def gemv(x: torch.Tensor, packed: torch.Tensor, codebook: torch.Tensor, bits: int, block_size: int,
         n: int, k: int, out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None,
         ws: torch.Tensor | None = None, ordered: bool = False) -> torch.Tensor:
    """y (M, n) = x (M, k) @ W.T for M <= 16, fused unpack + codebook gather + contraction.
    Launches on torch's current stream of x's device.  ordered=True: the launch does not start early
    (needed when `packed` or `codebook` were just written by earlier work of the stream)."""
    if not (x.is_cuda and packed.is_cuda and codebook.is_cuda):
        _need_cuda(x, packed, codebook)
    if x.dim() != 2 or x.shape[1] != k or not x.is_contiguous():
        raise RuntimeError(f"x must be a contiguous (M, {k}) tensor; got {tuple(x.shape)}")
    m = x.shape[0]
    xd = _DTYPE.get(x.dtype)
    if xd is None:
        raise RuntimeError(f"unsupported activation dtype {x.dtype}")
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype or x.dtype, device=x.device)
    dev = x.device.index
    if dev != torch.cuda.current_device():
        with torch.cuda.device(dev):
            return gemv(x, packed, codebook, bits, block_size, n, k, out=out, ws=ws, ordered=ordered)
    st = _raw_stream(dev) if _raw_stream is not None else torch.cuda.current_stream().cuda_stream
    if ws is None:
        ws = _workspaces.get((dev, st))
        if ws is None:
            ws = workspace(x.device, gemv_workspace_bytes(m, n, k, bits, block_size))
        elif ws.numel() < (32 << 20):       # a workspace of 32 MiB covers every shape the kernel accepts
            need = gemv_workspace_bytes(m, n, k, bits, block_size)
            if ws.numel() < need:
                ws = workspace(x.device, need)
    fn = _gemv_fn[1 if ordered else 0]
    if fn is None:
        fn = _gemv_fn[1 if ordered else 0] = _lib.lib().nb_gemv_ordered if ordered else _lib.lib().nb_gemv
    rc = fn(x.data_ptr(), xd, m, packed.data_ptr(), codebook.data_ptr(), _DTYPE[codebook.dtype], bits,
            block_size, n, k, out.data_ptr(), _DTYPE[out.dtype], ws.data_ptr(), ws.numel(), st)
    if rc:
        _lib.check(rc, "nb_gemv")
    return out


_gemv_fn = [None, None]

PRO_NONE, PRO_ADD_RMSNORM, PRO_SILU_MUL = 0, 1, 2


def gemv_fused(prologue: int, x: torch.Tensor, packed: torch.Tensor, codebook: torch.Tensor, bits: int, block_size: int,
               n: int, k: int, out: torch.Tensor, delta: torch.Tensor | None = None, norm_weight: torch.Tensor | None = None,
               eps: float = 0.0, x_out: torch.Tensor | None = None, ws: torch.Tensor | None = None) -> torch.Tensor:
    """nb_gemv with the decoder's element-wise step before it computed while the activations are staged.
    PRO_ADD_RMSNORM: x (M, k) fp32 residual, delta (M, k) or None, norm_weight (k); x + delta goes to x_out.
    PRO_SILU_MUL: x (M, 2k) fp32 = [gate | up].  M <= 8."""
    if not (x.is_cuda and packed.is_cuda and codebook.is_cuda):
        _need_cuda(x, packed, codebook)
    cols = 2 * k if prologue == PRO_SILU_MUL else k
    if x.dtype != torch.float32 or x.dim() != 2 or x.shape[1] != cols or not x.is_contiguous():
        raise RuntimeError(f"x must be a contiguous fp32 (M, {cols}) tensor; got {x.dtype} {tuple(x.shape)}")
    m = x.shape[0]
    for name, t in (("delta", delta), ("norm_weight", norm_weight), ("x_out", x_out)):
        if t is not None and (t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous()):
            raise RuntimeError(f"{name} must be a contiguous fp32 CUDA tensor")
    if ws is None:
        ws = workspace(x.device, gemv_workspace_bytes(m, n, k, bits, block_size))
    ptr = lambda t: t.data_ptr() if t is not None else None
    rc = _lib.lib().nb_gemv_fused(prologue, x.data_ptr(), ptr(delta), ptr(norm_weight), eps, ptr(x_out), m, packed.data_ptr(),
                                  codebook.data_ptr(), _DTYPE[codebook.dtype], bits, block_size, n, k, out.data_ptr(),
                                  _DTYPE[out.dtype], ws.data_ptr(), ws.numel(), _stream())
    if rc:
        _lib.check(rc, "nb_gemv_fused")
    return out


def gemv_stream(prologue: int, x: torch.Tensor, w_stream: torch.Tensor, bits: int, n: int, k: int, out: torch.Tensor,
                delta: torch.Tensor | None = None, norm_weight: torch.Tensor | None = None, eps: float = 0.0,
                x_out: torch.Tensor | None = None, swiglu: bool = False, single_term: bool = False,
                accumulate: bool = False) -> torch.Tensor:
    """One packed matvec of a dependent chain over the stream-layout copy of the weights (nb_gemv_stream): out (n) fp32
    = W . act(x), act as in gemv_fused (PRO_NONE: x of any float type; PRO_ADD_RMSNORM / PRO_SILU_MUL: fp32).
    swiglu: W is a [gate | up] matrix packed with row_mode 1 and out receives the n / 2 values silu(gate) * up.
    single_term: fp32 activations enter the tensor cores rounded to one fp16 value (11 significant bits) instead of as
    two fp16 terms (22 bits): half the MMAs, an error of a few 1e-4 of max |y| per matvec (4e-3 of max |logit| through the
    26-layer decoder).  accumulate: out += W act(x) (the residual update of a block; not together with swiglu)."""
    _need_cuda(x, w_stream, out)
    cols = 2 * k if prologue == PRO_SILU_MUL else k
    n_out = n // 2 if swiglu else n
    if x.numel() != cols or not x.is_contiguous() or out.dtype != torch.float32 or out.numel() != n_out or not out.is_contiguous():
        raise RuntimeError(f"gemv_stream needs one contiguous activation row of {cols} values and an fp32 output of {n_out}")
    if prologue != PRO_NONE and x.dtype != torch.float32:
        raise RuntimeError("the fused prologues take fp32 activations")
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().nb_gemv_stream(prologue, x.data_ptr(), _DTYPE[x.dtype], 0 if delta is None else delta.data_ptr(),
                                             0 if norm_weight is None else norm_weight.data_ptr(), float(eps),
                                             0 if x_out is None else x_out.data_ptr(), w_stream.data_ptr(), bits, n, k,
                                             out.data_ptr(), (1 if swiglu else 0) | (2 if single_term else 0) | (4 if accumulate else 0), _stream()),
                   "nb_gemv_stream")
    return out


_max_rows: dict = {}


def gemv_stream_max_rows(bits: int, k: int) -> int:
    """Activation rows one nb_gemv_stream_rows call takes for a matrix with k columns (8 at k = 2560, 3 at k = 6912)."""
    key = (bits, k)
    if key not in _max_rows:
        _max_rows[key] = int(_lib.lib().nb_gemv_stream_max_rows(bits, k))
    return _max_rows[key]


def gemv_stream_rows(prologue: int, x: torch.Tensor, w_stream: torch.Tensor, bits: int, n: int, k: int, out: torch.Tensor,
                     delta: torch.Tensor | None = None, norm_weight: torch.Tensor | None = None, eps: float = 0.0,
                     x_out: torch.Tensor | None = None, swiglu: bool = False) -> torch.Tensor:
    """gemv_stream for a few fp32 activation rows in one pass over the weights (nb_gemv_stream_rows): out (m, n) fp32 =
    act(x) W^T for x (m, k) — (m, 2k) with PRO_SILU_MUL.  More rows than gemv_stream_max_rows(bits, k) are split over
    several launches here.  swiglu: W is a [gate | up] matrix packed with row_mode 1 and out is (m, n / 2)."""
    _need_cuda(x, w_stream, out)
    cols = 2 * k if prologue == PRO_SILU_MUL else k
    n_out = n // 2 if swiglu else n
    if (x.dim() != 2 or x.shape[1] != cols or x.dtype != torch.float32 or not x.is_contiguous() or out.dtype != torch.float32
            or out.shape != (x.shape[0], n_out) or not out.is_contiguous()):
        raise RuntimeError(f"gemv_stream_rows needs contiguous fp32 x (m, {cols}) and out (m, {n_out})")
    for t in (delta, x_out):
        if t is not None and (t.dtype != torch.float32 or t.shape != (x.shape[0], k) or not t.is_contiguous()):
            raise RuntimeError(f"gemv_stream_rows: delta and x_out must be contiguous fp32 (m, {k})")
    m, step = x.shape[0], gemv_stream_max_rows(bits, k)
    if step < 1:
        raise RuntimeError(f"gemv_stream_rows: no row of {k} activations fits ({bits} bits)")
    with torch.cuda.device(x.device):
        for r0 in range(0, m, step):
            r1 = min(m, r0 + step)
            _lib.check(_lib.lib().nb_gemv_stream_rows(prologue, x[r0:r1].data_ptr(), r1 - r0,
                                                      0 if delta is None else delta[r0:r1].data_ptr(),
                                                      0 if norm_weight is None else norm_weight.data_ptr(), float(eps),
                                                      0 if x_out is None else x_out[r0:r1].data_ptr(), w_stream.data_ptr(), bits, n, k,
                                                      out[r0:r1].data_ptr(), 1 if swiglu else 0, _stream()), "nb_gemv_stream_rows")
    return out


def gemv_tp(prologue: int, x: torch.Tensor, packed: torch.Tensor, codebook: torch.Tensor, bits: int, block_size: int,
            n: int, k: int, exchange, out: torch.Tensor | None = None, gather: bool = False, push: bool = False,
            norm_weight: torch.Tensor | None = None, eps: float = 0.0, x_out: torch.Tensor | None = None,
            delta: torch.Tensor | None = None, ws: torch.Tensor | None = None) -> None:
    """nb_gemv_fused with the tensor-parallel all-reduce folded in: push sends the result to every
    rank's exchange buffer (comm.Exchange) instead of `out`; gather takes the residual delta as the sum
    of the vectors the ranks pushed last."""
    cols = 2 * k if prologue == PRO_SILU_MUL else k
    if not x.is_cuda or x.dtype != torch.float32 or x.dim() != 2 or x.shape[1] != cols or not x.is_contiguous():
        raise RuntimeError(f"x must be a contiguous fp32 CUDA (M, {cols}) tensor; got {x.dtype} {tuple(x.shape)}")
    m = x.shape[0]
    if ws is None:
        ws = workspace(x.device, gemv_workspace_bytes(m, n, k, bits, block_size))
    ptr = lambda t: t.data_ptr() if t is not None else None
    rc = _lib.lib().nb_gemv_tp(prologue, x.data_ptr(), ptr(delta), ptr(norm_weight), eps, ptr(x_out), m, packed.data_ptr(),
                               codebook.data_ptr(), _DTYPE[codebook.dtype], bits, block_size, n, k, ptr(out),
                               _DTYPE[out.dtype] if out is not None else 0, ws.data_ptr(), ws.numel(), exchange.buf.data_ptr(),
                               exchange.world, exchange.rank, exchange.max_count, int(gather), int(push), exchange.spin_limit,
                               _stream())
    if rc:
        _lib.check(rc, "nb_gemv_tp")


def exchange_gather(out: torch.Tensor, exchange, status: torch.Tensor) -> None:
    rc = _lib.lib().nb_exchange_gather(out.data_ptr(), out.numel(), exchange.buf.data_ptr(), exchange.world, exchange.rank,
                                       exchange.max_count, exchange.spin_limit, status.data_ptr(), _stream())
    if rc:
        _lib.check(rc, "nb_exchange_gather")


_prefill_ws: dict = {}


def prefill_workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Scratch for the dequantised bf16 weight of the prefill GEMM, one per (device, stream)."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream())
    ws = _prefill_ws.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _prefill_ws[key] = ws
    return ws


def gemm_prefill(x: torch.Tensor, packed: torch.Tensor, codebook: torch.Tensor, bits: int, block_size: int,
                 n: int, k: int, out_dtype: torch.dtype = torch.bfloat16, out: torch.Tensor | None = None) -> torch.Tensor:
    """y (M, n) = x (M, k) @ W.T on the tcgen05 tensor cores: W is dequantised once into the workspace, then
    the plain tensor-core kernel multiplies.  x bf16, fp16 or fp32; the library carries fp32 activations as two
    fp16 terms per element (about 22 significant bits, as in the GEMV) in adjacent operand rows and adds their
    results in the epilogue."""
    _need_cuda(x, packed, codebook)
    if x.dtype not in (torch.bfloat16, torch.float16, torch.float32) or x.dim() != 2 or x.shape[1] != k:
        raise RuntimeError(f"x must be a bf16, fp16 or fp32 (M, {k}) tensor; got {x.dtype} {tuple(x.shape)}")
    if not x.is_contiguous():
        x = x.contiguous()
    m = x.shape[0]
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else x.dtype
    if out is None and out_dtype == torch.float16:     # the kernel writes bf16 or fp32
        return gemm_prefill(x, packed, codebook, bits, block_size, n, k, out_dtype=torch.float32).half()
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype, device=x.device)
    l = _lib.lib()
    with torch.cuda.device(x.device):
        need = l.nb_prefill_workspace_bytes(m, n, k)
        ws = prefill_workspace(x.device, need)
        _lib.check(l.nb_gemm_prefill(x.data_ptr(), _DTYPE[x.dtype], m, packed.data_ptr(), codebook.data_ptr(), _DTYPE[codebook.dtype], bits,
                                     block_size, n, k, out.data_ptr(), _DTYPE[out.dtype], ws.data_ptr(), ws.numel(),
                                     _stream()), "nb_gemm_prefill")
    return out


def gemm_prefill_fused(x: torch.Tensor, w_stream: torch.Tensor, bits: int, n: int, k: int,
                       out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """y (M, n) = x (M, k) @ W.T with the dequantisation fused into the tcgen05 kernel; w_stream is the
    stream-layout copy of the packed weight (stream.stream_pack).  x fp16, bf16 or fp32; the library carries
    fp32 activations as two fp16 terms per element (rows 2i, 2i+1 of the operand) and adds their results."""
    _need_cuda(x, w_stream)
    if x.dim() != 2 or x.shape[1] != k:
        raise RuntimeError(f"x must be an (M, {k}) tensor; got {tuple(x.shape)}")
    if x.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        raise RuntimeError(f"unsupported activation dtype {x.dtype}")
    if not x.is_contiguous():
        x = x.contiguous()
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else x.dtype
    if out is None and out_dtype == torch.float16:     # the kernel writes bf16 or fp32
        return gemm_prefill_fused(x, w_stream, bits, n, k, out_dtype=torch.float32).half()
    m = x.shape[0]
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype, device=x.device)
    l = _lib.lib()
    with torch.cuda.device(x.device):
        need = int(l.nb_prefill_fused_workspace_bytes(m, n, k))
        ws = prefill_workspace(x.device, need)
        _lib.check(l.nb_gemm_prefill_fused(x.data_ptr(), _DTYPE[x.dtype], m, w_stream.data_ptr(), bits, n, k, out.data_ptr(),
                                           _DTYPE[out.dtype], ws.data_ptr(), ws.numel(), _stream()), "nb_gemm_prefill_fused")
    return out


def prefill_status(device) -> int:
    """Status word of the prefill workspace of the current stream (0, or NB_ERR_TIMEOUT); synchronises."""
    key = (torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device(), _stream())
    ws = _prefill_ws.get(key)
    return 0 if ws is None else int(ws[:4].view(torch.int32).item())


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """y = x @ w.T for bf16 x (M, K) and w (N, K) with the hand-written tcgen05 kernel."""
    _need_cuda(x, w)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.shape[1] != w.shape[1]:
        raise RuntimeError("gemm_bf16 needs bf16 x (M, K) and w (N, K)")
    m, k = x.shape
    n = w.shape[0]
    out = torch.empty(m, n, dtype=out_dtype, device=x.device)
    with torch.cuda.device(x.device):
        # the status word is the head of this stream's persistent prefill workspace: prefill_status() reads it
        status = prefill_workspace(x.device, 256)
        _lib.check(_lib.lib().nb_gemm_bf16(x.data_ptr(), w.data_ptr(), m, n, k, out.data_ptr(), _DTYPE[out_dtype],
                                           status.data_ptr(), _stream()), "nb_gemm_bf16")
    return out


# ---------------------------------------------------------------------- decode-step glue kernels
def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, w: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """x (B, C) fp32 += delta; out = rmsnorm(x) * w."""
    _lib.check(_lib.lib().nb_add_rmsnorm(x.data_ptr(), 0 if delta is None else delta.data_ptr(), w.data_ptr(), eps,
                                         out.data_ptr(), x.shape[0], x.shape[1], _stream()), "nb_add_rmsnorm")


def rope_kv_write(qkv, n_heads, head_dim, cos2, sin2, pos, k_cache, v_cache, q_out) -> None:
    _lib.check(_lib.lib().nb_rope_kv_write(qkv.data_ptr(), qkv.shape[0], n_heads, head_dim, cos2.data_ptr(), sin2.data_ptr(),
                                           pos.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), k_cache.shape[2],
                                           q_out.data_ptr(), _stream()), "nb_rope_kv_write")


def decode_attention(q, k_cache, v_cache, pos, out, out_offset: int) -> None:
    b, h, ctx, hd = k_cache.shape
    _lib.check(_lib.lib().nb_decode_attention(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), pos.data_ptr(), b, h, hd,
                                              ctx, out.data_ptr(), out.shape[1], out_offset, _stream()), "nb_decode_attention")


def decode_attention_rope(qkv, cos2, sin2, pos, k_cache, v_cache, out, out_offset: int) -> None:
    """RoPE + cache write + single-query attention in one launch."""
    b, h, ctx, hd = k_cache.shape
    _lib.check(_lib.lib().nb_decode_attention_rope(qkv.data_ptr(), cos2.data_ptr(), sin2.data_ptr(), pos.data_ptr(),
                                                   k_cache.data_ptr(), v_cache.data_ptr(), b, h, hd, ctx, out.data_ptr(),
                                                   out.shape[1], out_offset, _stream()), "nb_decode_attention_rope")


def prefill_attention(qkv: torch.Tensor, T: int, cos2, sin2, pos0: int, k_cache, v_cache, out: torch.Tensor,
                      out_offset: int = 0) -> None:
    """RoPE + cache write + causal attention of a T-token prompt chunk per sequence in one launch.
    qkv (B*T, 3*H*hd) fp32 contiguous; caches (B, H, ctx, hd) fp32; out (B*T, >= out_offset + H*hd) fp32."""
    b, h, ctx, hd = k_cache.shape
    for t in (qkv, k_cache, v_cache, out, cos2, sin2):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise RuntimeError("prefill_attention needs contiguous fp32 tensors")
    if qkv.numel() != b * T * 3 * h * hd:
        raise RuntimeError(f"prefill_attention: qkv has {qkv.numel()} values, expected {b}*{T}*3*{h}*{hd}")
    if cos2.shape[0] < pos0 + T or cos2.shape[-1] != hd:
        raise RuntimeError("prefill_attention: the rotary tables do not cover the positions")
    _lib.check(_lib.lib().nb_prefill_attention(qkv.data_ptr(), b, T, h, hd, cos2.data_ptr(), sin2.data_ptr(), pos0,
                                               k_cache.data_ptr(), v_cache.data_ptr(), ctx, out.data_ptr(), out.shape[-1],
                                               out_offset, _stream()), "nb_prefill_attention")


def lm_head_supported(table: torch.Tensor) -> bool:
    return table.is_cuda and table.dtype == torch.bfloat16 and table.is_contiguous() and table.shape[1] % 256 == 0 and table.shape[1] <= 3072


_head_scratch: dict = {}


def lm_head(x: torch.Tensor, delta: torch.Tensor | None, norm_weight: torch.Tensor | None, eps: float, table: torch.Tensor, cap: float,
            logits_out: torch.Tensor, token: torch.Tensor, pos: torch.Tensor | None = None) -> None:
    """One sequence: logits_out (V) = cap * tanh(table @ (rmsnorm(x + delta) * norm_weight) / cap), token = arg-max,
    pos += 1 (nb_lm_head: the bf16 table is read once, final norm, soft-cap and arg-max ride in the same two launches)."""
    _need_cuda(x, table, logits_out)
    v, c = table.shape
    if not lm_head_supported(table) or x.numel() != c or x.dtype != torch.float32 or not x.is_contiguous():
        raise RuntimeError("lm_head needs a contiguous bf16 (V, C) table with C a multiple of 256 up to 3072 and one fp32 row of C values")
    if logits_out.dtype != torch.float32 or logits_out.numel() != v or not logits_out.is_contiguous() or token.dtype != torch.int64:
        raise RuntimeError("lm_head needs a contiguous fp32 output of V values and an int64 token")
    for t in (delta, norm_weight):
        if t is not None and (t.dtype != torch.float32 or t.numel() != c or not t.is_contiguous()):
            raise RuntimeError("lm_head: delta and norm_weight must be contiguous fp32 vectors of C values")
    key = (x.device.index, torch.cuda.current_stream(x.device).cuda_stream)
    scratch = _head_scratch.get(key)
    if scratch is None:
        scratch = _head_scratch[key] = torch.empty(int(_lib.lib().nb_lm_head_scratch_bytes()), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().nb_lm_head(x.data_ptr(), 0 if delta is None else delta.data_ptr(),
                                         0 if norm_weight is None else norm_weight.data_ptr(), float(eps), table.data_ptr(), v, c,
                                         float(cap), logits_out.data_ptr(), token.data_ptr(), 0 if pos is None else pos.data_ptr(),
                                         scratch.data_ptr(), _stream()), "nb_lm_head")


def embed_rows(table: torch.Tensor, token: torch.Tensor, out: torch.Tensor) -> None:
    """out (B, C) fp32 = table[token] for a bf16 (V, C) table and int64 token (B,)."""
    if table.dtype != torch.bfloat16 or token.dtype != torch.int64 or out.dtype != torch.float32:
        raise RuntimeError("embed_rows needs a bf16 table, int64 tokens and an fp32 output")
    _lib.check(_lib.lib().nb_embed_rows(table.data_ptr(), token.data_ptr(), out.shape[0], table.shape[0], table.shape[1],
                                        out.data_ptr(), _stream()), "nb_embed_rows")


def softcap_argmax(logits: torch.Tensor, cap: float, logits_out: torch.Tensor, token: torch.Tensor,
                   pos: torch.Tensor | None = None) -> None:
    """logits_out = cap * tanh(logits / cap) (fp32); token[b] = argmax; pos += 1 (if given)."""
    if logits.dtype not in (torch.bfloat16, torch.float32) or not logits.is_contiguous() or token.dtype != torch.int64:
        raise RuntimeError("softcap_argmax needs contiguous bf16/fp32 logits and int64 tokens")
    _lib.check(_lib.lib().nb_softcap_argmax(logits.data_ptr(), _DTYPE[logits.dtype], logits.shape[0], logits.shape[1], cap,
                                            logits_out.data_ptr(), token.data_ptr(), pos.data_ptr() if pos is not None else None,
                                            _stream()), "nb_softcap_argmax")


def silu_mul(gu: torch.Tensor, out: torch.Tensor) -> None:
    _lib.check(_lib.lib().nb_silu_mul(gu.data_ptr(), gu.shape[0], out.shape[1], out.data_ptr(), _stream()), "nb_silu_mul")
