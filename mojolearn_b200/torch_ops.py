"""Device-resident entry points: CUDA torch tensors in, CUDA torch tensors out,
on the caller's current stream, no host copies.

torch is plumbing here (device memory, streams, the caching allocator that
provides the scratch); the arithmetic is the hand-written CUDA behind the C ABI.
The reference has no per-operation torch op (its adapter registers only
`torch.ops.mojolearn.train`, adapters/torch/registration.cpp:129-137), so these
mirror the signatures of `linalg.matmul*` and follow the adapter's conventions:
contiguity and dtype are checked, never fixed silently; a refusal raises with
the library's message.

`torch.ops.mojolearn_b200.matmul` / `.linear_w` are registered as custom ops so
the product can sit inside a torch program (fake-tensor shapes included).
"""
import ctypes

import torch

from . import _native
from .linalg import OP_NN, OP_NT, OP_TN, W_BF16, W_F32, W_INT8_EXP, W_INT8_SCALE, leaf_count

PLAN_AUTO, PLAN_FLAT, PLAN_T128, PLAN_T64, PLAN_DECODE, PLAN_T32, PLAN_T128X64, PLAN_SKINNY, PLAN_PACKED = -1, 0, 1, 2, 3, 4, 5, 6, 7


def _check(t, name, dtype):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError("%s must be a CUDA tensor" % name)
    if t.dtype != dtype:
        raise TypeError("%s must be %s, got %s (operands are never cast)" % (name, dtype, t.dtype))
    if not t.is_contiguous():
        raise ValueError("%s must be contiguous" % name)
    return t


def _vp(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def check_status(device=None):
    """Synchronise `device` and raise if a bounded device-side wait ran out since the last check (the word is
    cleared by the read). The device-pointer entry points are asynchronous and cannot report this themselves;
    callers that keep results on the device call this once where they would synchronise anyway."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    v = int(_native.lib().b200i_decode_status(index))
    if v != 0:
        raise _native.NativeError("mojolearn_b200: a bounded device-side wait ran out (status %d); results computed "
                                  "since the last check are incomplete" % v)


_W_DTYPES = {W_F32: torch.float32, W_BF16: torch.uint16, W_INT8_EXP: torch.int8, W_INT8_SCALE: torch.int8}


ACT_NONE, ACT_GELU_ERF, ACT_GELU_TANH, ACT_SILU = 0, 1, 2, 3
ACT_PAIR_SWIGLU, ACT_PAIR_GEGLU_ERF, ACT_PAIR_GEGLU_TANH = 4, 5, 6  # over interleaved (gate, up) weight rows: output [m, n / 2]


def product(a, b, bscale=None, wkind=W_F32, op=OP_NN, out=None, plan=PLAN_AUTO, group_leaves=0, bias=None, act=ACT_NONE):
    """C = op(a) . op(b) with b in weight storage `wkind`. `plan` forces an
    execution plan (tests); every plan gives the same bits. `bias` (one float32 per
    output column) and `act` are applied where the product stores its output: the
    words of the product followed by the separate bias and activation seams."""
    _check(a, "a", torch.float32)
    wdtype = _W_DTYPES[wkind]
    if wkind == W_BF16 and b.dtype in (torch.int16, torch.bfloat16):
        b = b.view(torch.uint16)
    _check(b, "b", wdtype)
    if a.dim() != 2 or b.dim() != 2:
        raise ValueError("operands must be 2-D")
    if op == OP_NN:
        (m, k), (k2, n) = a.shape, b.shape
    elif op == OP_NT:
        (m, k), (n, k2) = a.shape, b.shape
    elif op == OP_TN:
        (k, m), (k2, n) = a.shape, b.shape
    else:
        raise ValueError("unknown op %r" % (op,))
    if k != k2:
        raise ValueError("contracted extents disagree: %d and %d" % (k, k2))
    if bscale is not None:
        _check(bscale, "bscale", torch.int32 if wkind == W_INT8_EXP else torch.float32)
        if bscale.shape != (n,):
            raise ValueError("one exponent or scale per weight row")
    dev = a.device
    if b.device != dev:
        raise ValueError("operands live on different devices")
    n_out = n // 2 if act >= ACT_PAIR_SWIGLU else n  # a gated store activation folds each (gate, up) column pair into one
    if out is None:
        out = torch.empty((m, n_out), dtype=torch.float32, device=dev)
    else:
        _check(out, "out", torch.float32)
        if tuple(out.shape) != (m, n_out):
            raise ValueError("out must be (%d, %d)" % (m, n_out))
    lib = _native.lib()
    with torch.cuda.device(dev):
        ws_bytes = int(lib.b200i_plan_workspace_bytes(m, n, k, plan, group_leaves))
        ws = torch.empty((max(ws_bytes, 16),), dtype=torch.uint8, device=dev) if ws_bytes else None
        if bias is None and act == ACT_NONE:
            _native.call("b200i_gemm_w_plan", dev.index, _stream(dev), _vp(out), _vp(a), _vp(b), _vp(bscale), wkind, m, n, k,
                         op, plan, group_leaves, _vp(ws), ws_bytes)
        else:
            if bias is not None:
                _check(bias, "bias", torch.float32)
                if bias.shape != (n,):
                    raise ValueError("one bias word per output column")
            _native.call("b200i_gemm_w_epilogue", dev.index, _stream(dev), _vp(out), _vp(a), _vp(b), _vp(bscale), wkind, m, n, k,
                         op, _vp(bias), act, plan, group_leaves, _vp(ws), ws_bytes)
    return out


def product_nodes(a, b, bscale=None, wkind=W_F32, bias=None, act=ACT_NONE):
    """The NT product of `product` for a caller that folds leaf-group nodes itself (the gather after a column-sharded
    product). Returns (out, ws, nodes): with nodes == 1 `out` is the finished product; with nodes > 1 `out` is None
    and ws holds nodes x m x n float32 node words, to be finished by `PeerExchange.gather_nodes`."""
    _check(a, "a", torch.float32)
    if wkind == W_BF16 and b.dtype in (torch.int16, torch.bfloat16):
        b = b.view(torch.uint16)
    _check(b, "b", _W_DTYPES[wkind])
    (m, k), (n, k2) = a.shape, b.shape
    if k != k2:
        raise ValueError("contracted extents disagree: %d and %d" % (k, k2))
    if bscale is not None:
        _check(bscale, "bscale", torch.int32 if wkind == W_INT8_EXP else torch.float32)
    if bias is not None:
        _check(bias, "bias", torch.float32)
        if bias.shape != (n,):
            raise ValueError("one bias word per output column")
    dev = a.device
    n_out = n // 2 if act >= ACT_PAIR_SWIGLU else n
    out = torch.empty((m, n_out), dtype=torch.float32, device=dev)
    lib = _native.lib()
    nodes = ctypes.c_int64(1)
    with torch.cuda.device(dev):
        ws_bytes = int(lib.b200i_plan_workspace_bytes(m, n, k, PLAN_AUTO, 0))
        ws = torch.empty((max(ws_bytes, 16),), dtype=torch.uint8, device=dev) if ws_bytes else None
        _native.call("b200i_gemm_w_nodes", dev.index, _stream(dev), _vp(out), _vp(a), _vp(b), _vp(bscale), wkind, m, n, k, OP_NT,
                     _vp(bias), act, _vp(ws), ws_bytes, ctypes.byref(nodes))
    if nodes.value > 1:
        return None, ws, int(nodes.value)
    return out, None, 1


def matmul(a, b, *, transpose_a=False, transpose_b=False, out=None):
    if transpose_a and transpose_b:
        raise ValueError("both transposes are not an operation of the profile; compute (b @ a).T instead")
    op = OP_TN if transpose_a else (OP_NT if transpose_b else OP_NN)
    return product(a, b, None, W_F32, op, out)


def matmul_bf16(a, b_bits, *, transpose_a=False, transpose_b=False, out=None):
    if transpose_a and transpose_b:
        raise ValueError("both transposes are not an operation of the profile")
    if a.dtype in (torch.uint16, torch.int16):
        a = from_bf16(a)
    op = OP_TN if transpose_a else (OP_NT if transpose_b else OP_NN)
    return product(a, b_bits, None, W_BF16, op, out)


def linear_int8w(x, codes, exponents=None, scales=None, out=None):
    """x [m, k] float32 times an int8-stored weight [n, k] (per-row exponents, or
    per-row float32 scales as the extension): x @ W^T."""
    if (exponents is None) == (scales is None):
        raise ValueError("give exactly one of exponents or scales")
    if exponents is not None:
        return product(x, codes, exponents, W_INT8_EXP, OP_NT, out)
    return product(x, codes, scales, W_INT8_SCALE, OP_NT, out)


def to_bf16(x):
    _check(x, "x", torch.float32)
    out = torch.empty(x.shape, dtype=torch.uint16, device=x.device)
    if x.numel():
        with torch.cuda.device(x.device):
            _native.call("b200i_to_bf16", x.device.index, _stream(x.device), _vp(out), _vp(x), x.numel())
    return out


def from_bf16(bits):
    if bits.dtype in (torch.int16, torch.bfloat16):
        bits = bits.view(torch.uint16)
    _check(bits, "bits", torch.uint16)
    out = torch.empty(bits.shape, dtype=torch.float32, device=bits.device)
    if bits.numel():
        with torch.cuda.device(bits.device):
            _native.call("b200i_from_bf16", bits.device.index, _stream(bits.device), _vp(out), _vp(bits), bits.numel())
    return out


def quantize_int8(x):
    _check(x, "x", torch.float32)
    if x.dim() != 2:
        raise ValueError("x must be 2-D")
    rows, cols = x.shape
    codes = torch.empty((rows, cols), dtype=torch.int8, device=x.device)
    exps = torch.empty((rows,), dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        _native.call("b200i_quantize_int8", x.device.index, _stream(x.device), _vp(codes), _vp(exps), _vp(x), rows, cols)
    return codes, exps


def dequantize_int8(codes, exponents):
    _check(codes, "codes", torch.int8)
    _check(exponents, "exponents", torch.int32)
    rows, cols = codes.shape
    y = torch.empty((rows, cols), dtype=torch.float32, device=codes.device)
    with torch.cuda.device(codes.device):
        _native.call("b200i_dequantize_int8", codes.device.index, _stream(codes.device), _vp(y), _vp(codes), _vp(exponents),
                     rows, cols)
    return y


def matmul_int8(qa, ea, qb, eb):
    """int8i32.v1 at OP_NT on device tensors."""
    _check(qa, "qa", torch.int8)
    _check(qb, "qb", torch.int8)
    _check(ea, "ea", torch.int32)
    _check(eb, "eb", torch.int32)
    (m, k), (n, k2) = qa.shape, qb.shape
    if k != k2:
        raise ValueError("contracted extents disagree")
    c = torch.empty((m, n), dtype=torch.float32, device=qa.device)
    with torch.cuda.device(qa.device):
        _native.call("b200i_gemm_int8", qa.device.index, _stream(qa.device), _vp(c), _vp(qa), _vp(ea), _vp(qb), _vp(eb), m, n, k)
    return c


def matmul_int15(ah, al, ea, bh, bl, eb):
    """int15i64.v1 at OP_NT on device tensors: two int8 planes and one int32 exponent per row for each operand."""
    for t, name in ((ah, "ah"), (al, "al"), (bh, "bh"), (bl, "bl")):
        _check(t, name, torch.int8)
    _check(ea, "ea", torch.int32)
    _check(eb, "eb", torch.int32)
    (m, k), (n, k2) = ah.shape, bh.shape
    if k != k2 or al.shape != ah.shape or bl.shape != bh.shape:
        raise ValueError("planes of one operand must have one shape and the contracted extents must agree")
    c = torch.empty((m, n), dtype=torch.float32, device=ah.device)
    with torch.cuda.device(ah.device):
        _native.call("b200i_gemm_int15", ah.device.index, _stream(ah.device), _vp(c), _vp(ah), _vp(al), _vp(ea), _vp(bh), _vp(bl), _vp(eb), m, n, k)
    return c


# ---- torch.library registration ---------------------------------------------------------------

@torch.library.custom_op("mojolearn_b200::matmul", mutates_args=())
def _matmul_op(a: torch.Tensor, b: torch.Tensor, op: int) -> torch.Tensor:
    return product(a, b, None, W_F32, op)


@_matmul_op.register_fake
def _(a, b, op):
    m = a.shape[1] if op == OP_TN else a.shape[0]
    n = b.shape[0] if op == OP_NT else b.shape[1]
    return a.new_empty((m, n))


@torch.library.custom_op("mojolearn_b200::linear_w", mutates_args=())
def _linear_w_op(x: torch.Tensor, w: torch.Tensor, wscale: torch.Tensor, wkind: int) -> torch.Tensor:
    return product(x, w, wscale if wkind in (W_INT8_EXP, W_INT8_SCALE) else None, wkind, OP_NT)


@_linear_w_op.register_fake
def _(x, w, wscale, wkind):
    return x.new_empty((x.shape[0], w.shape[0]))
