"""Programs for the persistent multi-matrix kernel (csrc/nb_stream.cu): one launch runs a whole
decode step of the packed decoder, or any group of packed matvecs, with the weights streamed
through shared memory in a tile-major copy of the packed matrices.

The reference issues the same work as one library launch per operation and one host round trip per
token (inference/generate_torch.py:150-162, :307-311); this module only assembles the operation
list (host code) and hands it to nb_stream_run.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib, ops
from ._lib import NB_BF16, NB_F16, NB_F32

SOP_GEMV, SOP_ATTN, SOP_HEAD, SOP_ARGMAX, SOP_REDUCE = 1, 2, 3, 4, 5
SPRO_VEC, SPRO_EMBED_NORM, SPRO_ADD_NORM, SPRO_ATTN_MERGE = 0, 1, 2, 3
SEPI_STORE, SEPI_SLOTS, SEPI_SWIGLU = 0, 1, 2
SOPF_WAIT_PREV, SOPF_ALIGN, SOPF_REUSE_X = 1, 2, 4
STATUS_WORD = 513            # uint32 index of the status word in the state buffer

_DT = {torch.float32: NB_F32, torch.float16: NB_F16, torch.bfloat16: NB_BF16}


class StreamOp(ctypes.Structure):
    """Mirror of nb_stream_op (include/nativebit_b200.h)."""
    _fields_ = [("kind", ctypes.c_int32), ("flags", ctypes.c_int32), ("pro", ctypes.c_int32), ("epi", ctypes.c_int32),
                ("p", ctypes.c_void_p * 8), ("i", ctypes.c_int32 * 16), ("f", ctypes.c_float * 4)]


def _op(kind, flags=0, pro=0, epi=0, p=(), i=(), f=()) -> StreamOp:
    o = StreamOp()
    o.kind, o.flags, o.pro, o.epi = kind, flags, pro, epi
    for j, t in enumerate(p):
        o.p[j] = None if t is None else (t if isinstance(t, int) else t.data_ptr())
    for j, v in enumerate(i):
        o.i[j] = int(v)
    for j, v in enumerate(f):
        o.f[j] = float(v)
    return o


def n_ctas() -> int:
    return int(_lib.lib().nb_stream_ctas())


def n_slots(n: int, k: int) -> int:
    """Partial-sum slots a matvec with the slot epilogue writes per output (CTAs that can share a row tile)."""
    return int(_lib.lib().nb_stream_slots(n, k, n_ctas()))


def stream_pack(packed: torch.Tensor, codebook: torch.Tensor, bits: int, n: int, k: int, row_mode: int = 0) -> torch.Tensor:
    """Tile-major copy of a packed (n, k) matrix for the persistent kernel.  row_mode 1: a fused
    [gate | up] matrix whose gate and up rows are interleaved in groups of 8 (SwiGLU epilogue)."""
    if not (packed.is_cuda and codebook.is_cuda):
        raise RuntimeError("stream_pack needs CUDA tensors")
    l = _lib.lib()
    nbytes = int(l.nb_stream_packed_bytes(n, k, bits))
    if nbytes == 0:
        raise RuntimeError(f"the persistent kernel does not support N={n} K={k} bits={bits}")
    out = torch.empty(nbytes, dtype=torch.uint8, device=packed.device)
    with torch.cuda.device(packed.device):
        _lib.check(l.nb_stream_pack(packed.data_ptr(), codebook.data_ptr(), _DT[codebook.dtype], bits, n, k, row_mode,
                                    out.data_ptr(), ops._stream()), "nb_stream_pack")
    return out


class StreamProgram:
    """A list of operations, validated by the library at every launch and kept in device memory."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.ops: list[StreamOp] = []
        self.keep: list = []                 # tensors the operations point to
        self.state = torch.zeros(int(_lib.lib().nb_stream_state_bytes()), dtype=torch.uint8, device=self.device)
        self._host = None
        self._dev = None

    def add(self, op: StreamOp, *tensors) -> None:
        self.ops.append(op)
        self.keep.extend(tensors)
        self._host = None

    def _finalize(self) -> None:
        arr = (StreamOp * len(self.ops))(*self.ops)
        self._host = arr
        raw = bytes(arr)
        self._dev = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(self.device)

    def run(self, spin_limit: int = 0) -> None:
        if self._host is None:
            self._finalize()
        with torch.cuda.device(self.device):
            rc = _lib.lib().nb_stream_run(self._host, self._dev.data_ptr(), len(self.ops), self.state.data_ptr(), spin_limit,
                                          ops._stream())
        if rc:
            _lib.check(rc, "nb_stream_run")

    def status(self) -> int:
        """0, or NB_ERR_TIMEOUT (6) if a bounded wait ran out; synchronises."""
        return int(self.state.view(torch.int32)[STATUS_WORD].item())

    # ------------------------------------------------------------------ common operations
    def gemv_vec(self, w_stream, n, k, bits, x, out, *, wait=False, reuse_x=False, slots=None):
        """y = W x for a plain activation vector x (k,).  out: (n,) tensor (whole 16-row tiles per CTA), or
        with `slots` = number of slots: an fp32 (slots, n) tensor of partial sums (rows split freely)."""
        flags = (SOPF_WAIT_PREV if wait else 0) | (SOPF_REUSE_X if reuse_x else 0) | (0 if slots else SOPF_ALIGN)
        self.add(_op(SOP_GEMV, flags, SPRO_VEC, SEPI_SLOTS if slots else SEPI_STORE, p=(w_stream, x, None, None, out),
                     i=(n, k, bits, _DT[x.dtype], _DT[out.dtype], 0, slots or 0, 0, n)), w_stream, x, out)

    def reduce(self, slots_t, n, out, *, wait=False):
        self.add(_op(SOP_REDUCE, SOPF_WAIT_PREV if wait else 0, p=(None, slots_t, None, None, out),
                     i=(n, 0, 0, 0, _DT[out.dtype], slots_t.shape[0], 0, slots_t.shape[1])), slots_t, out)


def build_decode_program(model, session) -> StreamProgram:
    """The decode step of a single-sequence session as one program: per layer qkv (embedding or residual
    add + RMSNorm in its prologue), attention, out_proj, gate_up (SwiGLU in its epilogue), down; then the
    final norm + LM head + soft-cap and the greedy argmax.  Reads session.token / session.pos, writes
    session.logits, the next token and the incremented position."""
    cfg = model.config
    dev = model.embedding.device
    if session.B != 1:
        raise RuntimeError("the persistent decode step handles one sequence")
    if model.embedding.dtype != torch.bfloat16:
        raise RuntimeError("the persistent decode step needs a bf16 embedding table")
    C, hd, Hl, bits = cfg.n_embd, cfg.head_dim, model.heads_local, cfg.bits
    G = n_ctas()
    prog = StreamProgram(dev)
    f32 = dict(dtype=torch.float32, device=dev)
    sw = stream_weights(model)
    blk0 = model.blocks[0]
    n_qkv, k_o, n_gu, k_d = blk0.qkv.out_features, blk0.out_proj.in_features, blk0.gate_up.out_features, blk0.down.in_features
    s_qkv, s_o, s_d = n_slots(n_qkv, C), n_slots(C, k_o), n_slots(C, k_d)
    qkv_slots = torch.zeros(s_qkv, n_qkv, **f32)
    o_slots = torch.zeros(s_o, C, **f32)
    d_slots = torch.zeros(s_d, C, **f32)
    act = torch.zeros(n_gu // 2, **f32)
    splits = max(1, min(G // Hl, 16))
    att_part = torch.zeros(Hl * splits, hd + 2, **f32)
    cand = torch.zeros(2 * G, **f32)
    eps = cfg.norm_eps
    for l, blk in enumerate(model.blocks):
        k_buf, v_buf, _ = session.caches[l]
        w = sw[l]
        if l == 0:
            prog.add(_op(SOP_GEMV, 0, SPRO_EMBED_NORM, SEPI_SLOTS, p=(w["qkv"], model.embedding, session.token, blk.ln1, qkv_slots),
                         i=(n_qkv, C, bits, 0, 0, 0, s_qkv, 0, n_qkv, 0, 0, 0, 0, model.embedding.shape[0]), f=(eps,)), w["qkv"], blk.ln1)
        else:
            prog.add(_op(SOP_GEMV, SOPF_WAIT_PREV, SPRO_ADD_NORM, SEPI_SLOTS, p=(w["qkv"], d_slots, None, blk.ln1, qkv_slots),
                         i=(n_qkv, C, bits, 0, 0, s_d, s_qkv, C, n_qkv), f=(eps,)), w["qkv"], blk.ln1)
        prog.add(_op(SOP_ATTN, SOPF_WAIT_PREV, p=(qkv_slots, model.cos2, model.sin2, session.pos, k_buf, v_buf, att_part),
                     i=(Hl, hd, cfg.context_len, splits, 0, s_qkv, 0, n_qkv)), k_buf, v_buf)
        prog.add(_op(SOP_GEMV, SOPF_WAIT_PREV, SPRO_ATTN_MERGE, SEPI_SLOTS, p=(w["out_proj"], att_part, None, None, o_slots),
                     i=(C, k_o, bits, 0, 0, 0, s_o, 0, C, Hl, splits, hd, model.o_col0)), w["out_proj"])
        prog.add(_op(SOP_GEMV, SOPF_WAIT_PREV | SOPF_ALIGN, SPRO_ADD_NORM, SEPI_SWIGLU, p=(w["gate_up"], o_slots, None, blk.ln2, act),
                     i=(n_gu, C, bits, 0, 0, s_o, 0, C, 0), f=(eps,)), w["gate_up"], blk.ln2)
        prog.add(_op(SOP_GEMV, SOPF_WAIT_PREV, SPRO_VEC, SEPI_SLOTS, p=(w["down"], act, None, None, d_slots),
                     i=(C, k_d, bits, NB_F32, 0, 0, s_d, 0, C)), w["down"])
    V = model.embedding.shape[0]
    prog.add(_op(SOP_HEAD, SOPF_WAIT_PREV, p=(model.embedding, d_slots, None, model.ln_f, session.logits, cand),
                 i=(V, C, 0, 0, 0, s_d, 0, C, 0), f=(eps, cfg.logit_cap)), model.ln_f)
    prog.add(_op(SOP_ARGMAX, SOPF_WAIT_PREV, p=(cand, session.token, session.pos), i=(G,)))
    prog.keep.extend([qkv_slots, o_slots, d_slots, act, att_part, cand, session.token, session.pos, session.logits,
                      model.embedding, model.cos2, model.sin2])
    return prog


def stream_weights(model) -> list[dict]:
    """Tile-major copies of every packed matrix of the model (built once, cached on the model)."""
    cached = getattr(model, "_stream_weights", None)
    if cached is not None:
        return cached
    out = []
    for blk in model.blocks:
        d = {name: getattr(blk, name).stream_weight() for name in ("qkv", "out_proj", "down")}   # shared with the prefill kernel
        d["gate_up"] = blk.gate_up.stream_weight(1)
        out.append(d)
    torch.cuda.synchronize(model.embedding.device)
    model._stream_weights = out
    return out


def stream_supported(model, batch_size: int) -> bool:
    cfg = model.config
    blk = model.blocks[0] if len(model.blocks) else None
    return (blk is not None and batch_size == 1 and model.tp_size == 1 and cfg.block_size == 128 and cfg.bits in (2, 3, 4)
            and model.embedding.dtype == torch.bfloat16 and cfg.n_embd % 128 == 0
            and cfg.head_dim % 4 == 0 and cfg.head_dim <= 128 and blk.gate_up.out_features % 16 == 0
            and max(blk.down.in_features, blk.out_proj.in_features, cfg.n_embd) <= 7168 and cfg.n_embd <= 2560
            and 5 * cfg.n_layers + 2 <= int(_lib.lib().nb_stream_max_ops()))


class GroupItem(ctypes.Structure):
    """Mirror of nb_group_item (include/nativebit_b200.h)."""
    _fields_ = [("w", ctypes.c_void_p), ("x", ctypes.c_void_p), ("y", ctypes.c_void_p),
                ("n", ctypes.c_int32), ("k", ctypes.c_int32), ("x_dtype", ctypes.c_int32), ("y_dtype", ctypes.c_int32),
                ("m", ctypes.c_int32), ("reserved", ctypes.c_int32)]


class MatvecGroup:
    """Independent packed matvecs y_i = W_i x_i at batch 1, executed by ONE launch (nb_group_run): the row
    tiles of all matrices are dealt out to the CTAs by weight bytes and every warp computes whole 16-row tiles,
    so the weights of all matrices stream through the SMs back to back with no launch or operation boundary
    between them.  items: (PackedLinear, x (k,) or (m, k), out (n,) or (m, n)) triples with up to 8 activation rows
    (16-bit activations for more than one); matrices that read the same x share its staged copy.  The reference runs one library launch per matrix
    (inference/triton_kernel.py:240-256)."""

    def __init__(self, items, device=None):
        items = list(items)
        if not items:
            raise RuntimeError("MatvecGroup needs at least one matvec")
        dev = torch.device(device) if device is not None else items[0][1].device
        l = _lib.lib()
        if len(items) > int(l.nb_group_max_items()):
            raise RuntimeError(f"at most {int(l.nb_group_max_items())} matvecs per launch")
        bits = items[0][0].bits
        arr = (GroupItem * len(items))()
        self.keep = []
        for i, (lin, x, out) in enumerate(items):
            if lin.block_size != 128 or lin.bits != bits:
                raise RuntimeError("MatvecGroup needs block size 128 and one index width for all matrices")
            m = x.numel() // lin.in_features
            if (x.numel() != m * lin.in_features or out.numel() != m * lin.out_features or m < 1 or not x.is_contiguous()
                    or not out.is_contiguous()):
                raise RuntimeError("MatvecGroup needs contiguous (m, k) activations and (m, n) outputs per matrix")
            w = lin.stream_weight()
            arr[i].w, arr[i].x, arr[i].y = w.data_ptr(), x.data_ptr(), out.data_ptr()
            arr[i].n, arr[i].k, arr[i].x_dtype, arr[i].y_dtype = lin.out_features, lin.in_features, _DT[x.dtype], _DT[out.dtype]
            arr[i].m = m
            self.keep.extend((w, x, out))
        nbytes = int(l.nb_group_plan_bytes(arr, len(items)))
        self._plan_host = ctypes.create_string_buffer(nbytes)
        _lib.check(l.nb_group_build(arr, len(items), bits, self._plan_host, nbytes), "nb_group_build")
        self._plan_dev = torch.frombuffer(bytearray(self._plan_host.raw), dtype=torch.uint8).to(dev)
        self.device = dev
        self.n_matvecs = len(items)

    def run(self) -> None:
        with torch.cuda.device(self.device):
            rc = _lib.lib().nb_group_run(self._plan_dev.data_ptr(), self._plan_host, ops._stream())
        if rc:
            _lib.check(rc, "nb_group_run")

    def check(self) -> None:
        """Nothing in this launch can time out (no flags, no barriers between CTAs): kept for symmetry with
        StreamProgram."""
        return None
