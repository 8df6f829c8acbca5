"""jasmine_b200 — Python plumbing over libjasmine_b200.so (the C ABI in include/jasmine_b200.h).

The product is the CUDA library and the C++20 headers under include/jasmine/.
This package only loads the library with ctypes and wraps torch tensors (used
for device memory, streams and torch.distributed) into the C structs, for the
tests and bench.py.  There is no CPU or eager fallback: when the shared library
is missing, `lib()` raises.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "libjasmine_b200.so"

# jsm_status
OK, INVALID_ARG, SHAPE, OOM, CUDA, NCCL, TIMEOUT, UNSUPPORTED = range(8)
STATUS_NAMES = ["OK", "INVALID_ARG", "SHAPE", "OOM", "CUDA", "NCCL", "TIMEOUT", "UNSUPPORTED"]
# jsm_dtype
F32, BF16, I32 = 0, 1, 2
# jsm_op
(OP_LEAF, OP_IMM, OP_ADD, OP_SUB, OP_MUL, OP_DIV, OP_GT, OP_LT, OP_EXP, OP_SIGMOID, OP_POW, OP_SQRT, OP_NEG,
 OP_RELU, OP_GELU, OP_SILU, OP_TANH) = range(17)
# jsm_rows_kind
ROWS_SUM, ROWS_MAX, ROWS_MEAN, ROWS_ARGMAX, ROWS_SOFTMAX, ROWS_LAYERNORM, ROWS_RMSNORM = range(7)
PAGE_SIZE = 64


class JsmError(RuntimeError):
    def __init__(self, status: int, msg: str):
        super().__init__(f"jasmine_b200: {STATUS_NAMES[status] if 0 <= status < 8 else status}: {msg}")
        self.status = status


class Mat(C.Structure):
    _fields_ = [("data", C.c_void_p), ("rows", C.c_int32), ("cols", C.c_int32), ("row_stride", C.c_int64),
                ("col_stride", C.c_int64), ("dtype", C.c_int32)]


class Instr(C.Structure):
    _fields_ = [("op", C.c_int32), ("arg", C.c_int32), ("imm", C.c_float)]


class ModelConfig(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("d_model", C.c_int32), ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("d_ffn", C.c_int32), ("vocab", C.c_int32), ("max_batch", C.c_int32),
                ("max_context", C.c_int32), ("norm_eps", C.c_float), ("rope_theta", C.c_float),
                ("tp_rank", C.c_int32), ("tp_size", C.c_int32)]


ALLREDUCE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.c_void_p)

# every symbol include/jasmine_b200.h declares: (restype, argtypes)
_vp, _i, _f, _sz, _u64, _i64 = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_uint64, C.c_int64
SYMBOLS = {
    "jsm_last_error": (C.c_char_p, []),
    "jsm_version": (_i, []),
    "jsm_device_count": (_i, [C.POINTER(_i)]),
    "jsm_launch_count": (_u64, []),
    "jsm_check_device_errors": (_i, [_vp]),
    "jsm_malloc": (_i, [C.POINTER(_vp), _sz]),
    "jsm_free": (_i, [_vp]),
    "jsm_upload": (_i, [_vp, _vp, _sz, _vp]),
    "jsm_download": (_i, [_vp, _vp, _sz, _vp]),
    "jsm_memset": (_i, [_vp, _i, _sz, _vp]),
    "jsm_stream_sync": (_i, [_vp]),
    "jsm_fill": (_i, [_vp, _i, _sz, _u64, _u64, _i, _f, _f, _vp]),
    "jsm_fill_host": (_i, [_vp, _i, _sz, _u64, _u64, _i, _f, _f]),
    "jsm_convert": (_i, [_vp, _i, _vp, _i, _sz, _vp]),
    "jsm_eval_elementwise": (_i, [C.POINTER(Instr), _i, C.POINTER(Mat), _i, Mat, _vp]),
    "jsm_eval_rows": (_i, [_i, _i, C.POINTER(Instr), _i, C.POINTER(Mat), _i, _vp, _vp, _f, Mat, _vp]),
    "jsm_eval_full": (_i, [_i, C.POINTER(Instr), _i, C.POINTER(Mat), _i, Mat, _vp]),
    "jsm_dot_f32": (_i, [Mat, Mat, C.POINTER(Mat), _i, C.POINTER(Mat), Mat, _vp]),
    "jsm_linear_bf16": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp]),
    "jsm_linear_packed_bytes": (_sz, [_i, _i, _i]),
    "jsm_linear_packed_plan": (_i, [_i, _i, _i, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)]),
    "jsm_trace_begin": (_i, [_i]),
    "jsm_trace_end": (_i, [_vp, _i, C.POINTER(_i), C.POINTER(_i)]),
    "jsm_linear_pack": (_i, [_vp, _i, _i, _i, _vp, _vp]),
    "jsm_linear_packed_reserve": (_i, [_i, _i, _i]),
    "jsm_linear_unpack": (_i, [_vp, _i, _i, _i, _vp, _vp]),
    "jsm_linear_bf16_packed": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp]),
    "jsm_linear_bf16_packed_chained": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp]),
    "jsm_rope_table": (_i, [_vp, _i, _i, _f, _i, _vp]),
    "jsm_rope_apply": (_i, [_vp, _vp, _i, _vp, _i, _i, _vp, _i, _vp]),
    "jsm_rope_apply_qk": (_i, [_vp, _vp, _i, _vp, _vp, _i, _i, _vp, _i, _vp, _i, _vp]),
    "jsm_attn_prefill": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _i, _vp]),
    "jsm_kv_append": (_i, [_vp, _vp, _i, _vp, _vp, _i64, _vp, _vp, _i, _i, _i, _vp, _vp]),
    "jsm_attn_decode_scratch_bytes": (_sz, [_i, _i, _i, _i]),
    "jsm_attn_decode_scratch_bytes_max": (_sz, [_i, _i, _i, _i]),
    "jsm_attn_decode": (_i, [_vp, _i64, _vp, _vp, _i, _vp, _i, _i, _i, _i, _f, _vp, _i, _vp, _vp, _vp]),
    "jsm_attn_decode_append": (_i, [_vp, _i64, _vp, _vp, _i64, _vp, _vp, _i, _vp, _i, _i, _i, _i, _f, _vp, _i, _vp, _vp, _vp, _vp]),
    "jsm_attn_decode_static_scratch": (_i, [_vp, _i64, _vp, _vp, _i, _vp, _i, _i, _i, _i, _f, _vp, _i, _vp, _vp]),
    "jsm_embedding": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "jsm_add_norm": (_i, [_i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _f, _i, _i, _vp]),
    "jsm_llama_create": (_i, [C.POINTER(ModelConfig), _u64, C.POINTER(_vp)]),
    "jsm_llama_destroy": (_i, [_vp]),
    "jsm_llama_set_allreduce": (_i, [_vp, ALLREDUCE_FN, _vp]),
    "jsm_llama_tp_region": (_i, [_vp, C.POINTER(_vp), C.POINTER(_sz)]),
    "jsm_llama_tp_connect": (_i, [_vp, C.POINTER(_vp)]),
    "jsm_tp_region_bytes": (_sz, [_i, _i]),
    "jsm_tp_inband_slot_offset": (_sz, [_i, _i, _i, _i]),
    "jsm_tp_set_wait_limit_ms": (_i, [_i]),
    "jsm_tp_allreduce_add_norm": (_i, [C.POINTER(_vp), _i, _i, _i, _i, _vp, _i, _i, _vp, _vp, _f, _i, _i, _vp]),
    "jsm_tp_linear_push": (_i, [C.POINTER(_vp), _i, _i, _i, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _vp]),
    "jsm_tp_linear_reduce": (_i, [_vp, _i, _i, _i, _i, _vp, _i, _i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _f, _vp]),
    "jsm_tp_argmax_exchange": (_i, [C.POINTER(_vp), _i, _i, _i, _i, _vp, _i, _i, _vp, _vp, _vp, _i, _vp]),
    "jsm_ipc_export": (_i, [_vp, C.c_char_p]),
    "jsm_ipc_import": (_i, [C.c_char_p, C.POINTER(_vp)]),
    "jsm_ipc_close": (_i, [_vp]),
    "jsm_sample": (_i, [_vp, C.c_int64, C.c_int, C.c_int, C.c_float, C.c_int, C.c_float, C.c_uint64, C.c_uint64, _vp, _vp]),
    "jsm_llama_weight": (_i, [_vp, C.c_char_p, C.POINTER(_vp), C.POINTER(_sz)]),
    "jsm_llama_set_weight": (_i, [_vp, C.c_char_p, _vp, _sz, _vp]),
    "jsm_llama_save": (_i, [_vp, C.c_char_p]),
    "jsm_llama_load": (_i, [_vp, C.c_char_p]),
    "jsm_llama_prefill": (_i, [_vp, _vp, _i, _i, _vp, _vp, _vp]),
    "jsm_llama_decode_step": (_i, [_vp, _vp, _i, _vp, _vp, _vp]),
    "jsm_llama_decode_step_host": (_i, [_vp, _vp, _i, _vp, _vp, _vp]),
    "jsm_llama_create_paged": (_i, [C.POINTER(ModelConfig), _u64, _i, C.POINTER(_vp)]),
    "jsm_llama_seq_admit": (_i, [_vp, _vp, _i, C.POINTER(_i), _vp, _vp, _vp]),
    "jsm_llama_step_active": (_i, [_vp, _vp, _vp, _vp, _vp]),
    "jsm_llama_seq_retire": (_i, [_vp, _i, C.POINTER(_i), _vp]),
    "jsm_llama_pool_state": (_i, [_vp, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)]),
    "jsm_llama_set_context": (_i, [_vp, _i, _i]),
    "jsm_llama_reset": (_i, [_vp]),
    "jsm_llama_step_bytes": (_i, [_vp, C.POINTER(_u64), C.POINTER(_u64)]),
}

_lib = None


def lib() -> C.CDLL:
    """Load libjasmine_b200.so (once).  Raises when it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise JsmError(CUDA, f"{LIB_PATH} is missing: build it with `python -m jasmine_b200.build`")
        L = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != OK:
        raise JsmError(status, lib().jsm_last_error().decode(errors="replace"))


# ---- torch plumbing ------------------------------------------------------------
def _torch():
    import torch
    return torch


def stream_ptr() -> int:
    return _torch().cuda.current_stream().cuda_stream


def dtype_of(t) -> int:
    torch = _torch()
    return {torch.float32: F32, torch.bfloat16: BF16, torch.int32: I32}[t.dtype]


def mat(t, rows: int | None = None, cols: int | None = None) -> Mat:
    """A 2-D torch tensor (any strides, i.e. views and transposes) as a jsm_mat."""
    if t.dim() == 1:
        t = t.unsqueeze(0)
    assert t.dim() == 2
    return Mat(t.data_ptr(), t.shape[0], t.shape[1], t.stride(0), t.stride(1), dtype_of(t))


def program(instrs):
    """[(op, arg_or_imm), ...] -> (Instr array, n).  LEAF takes a leaf index, IMM/POW a float."""
    arr = (Instr * len(instrs))()
    for k, ins in enumerate(instrs):
        op = ins[0]
        a = ins[1] if len(ins) > 1 else 0
        if op in (OP_IMM, OP_POW):
            arr[k] = Instr(op, 0, float(a))
        else:
            arr[k] = Instr(op, int(a), 0.0)
    return arr, len(instrs)


def _leaves(ts):
    arr = (Mat * max(1, len(ts)))()
    for k, t in enumerate(ts):
        arr[k] = mat(t)
    return arr, len(ts)


def eval_elementwise(instrs, leaves, out):
    p, n = program(instrs)
    l, nl = _leaves(leaves)
    check(lib().jsm_eval_elementwise(p, n, l, nl, mat(out), stream_ptr()))
    return out


def eval_rows(kind, axis, instrs, leaves, out, gain=None, bias=None, eps=0.0):
    p, n = program(instrs)
    l, nl = _leaves(leaves)
    check(lib().jsm_eval_rows(kind, axis, p, n, l, nl, gain.data_ptr() if gain is not None else None,
                              bias.data_ptr() if bias is not None else None, eps, mat(out), stream_ptr()))
    return out


def eval_full(kind, instrs, leaves, out):
    p, n = program(instrs)
    l, nl = _leaves(leaves)
    check(lib().jsm_eval_full(kind, p, n, l, nl, mat(out), stream_ptr()))
    return out


def dot_f32(A, B, out, bias=None, epilogue=0, residual=None):
    b = mat(bias) if bias is not None else None
    r = mat(residual) if residual is not None else None
    check(lib().jsm_dot_f32(mat(A), mat(B), C.byref(b) if b is not None else None, epilogue,
                            C.byref(r) if r is not None else None, mat(out), stream_ptr()))
    return out


def linear_bf16(X, W, out, bias=None, epilogue=0, residual=None):
    T, K = X.shape
    N = out.shape[1]
    check(lib().jsm_linear_bf16(X.data_ptr(), W.data_ptr(), bias.data_ptr() if bias is not None else None, epilogue,
                                residual.data_ptr() if residual is not None else None, out.data_ptr(), dtype_of(out),
                                T, N, K, stream_ptr()))
    return out


def linear_pack(W, N: int, paired: bool = False):
    """Packs a row-major bf16 weight matrix ([N, K], or [2N, K] gate rows then up rows when paired) once."""
    torch = _torch()
    K = W.shape[1]
    packed = torch.empty(lib().jsm_linear_packed_bytes(N, K, int(paired)), dtype=torch.uint8, device=W.device)
    check(lib().jsm_linear_pack(W.data_ptr(), N, K, int(paired), packed.data_ptr(), stream_ptr()))
    return packed


def linear_unpack(packed, N: int, K: int, paired: bool = False):
    torch = _torch()
    W = torch.zeros((2 * N if paired else N), K, dtype=torch.bfloat16, device=packed.device)
    check(lib().jsm_linear_unpack(packed.data_ptr(), N, K, int(paired), W.data_ptr(), stream_ptr()))
    return W


def linear_bf16_packed(X, packed, out, bias=None, epilogue=0, residual=None, chained=False):
    T, K = X.shape
    N = out.shape[1]
    fn = lib().jsm_linear_bf16_packed_chained if chained else lib().jsm_linear_bf16_packed
    check(fn(X.data_ptr(), packed.data_ptr(), bias.data_ptr() if bias is not None else None, epilogue,
             residual.data_ptr() if residual is not None else None, out.data_ptr(), dtype_of(out), T, N, K, stream_ptr()))
    return out


def rope_table(mode: int, d: int, theta: float, max_pos: int, device="cuda"):
    torch = _torch()
    t = torch.empty(max_pos, d // 2, 4, dtype=torch.float32, device=device)
    check(lib().jsm_rope_table(t.data_ptr(), mode, d, theta, max_pos, stream_ptr()))
    return t


def rope_apply(x, table, d, n_heads, positions=None, out=None):
    torch = _torch()
    out = torch.empty_like(x) if out is None else out
    check(lib().jsm_rope_apply(x.data_ptr(), out.data_ptr(), dtype_of(x), table.data_ptr(), d, n_heads,
                               positions.data_ptr() if positions is not None else None, x.shape[0], stream_ptr()))
    return out


def rope_apply_qk(q, k, table, d, Hq, Hkv, positions=None, q_out=None, k_out=None):
    """Queries and keys rotated by one launch (jsm_rope_apply_qk)."""
    torch = _torch()
    q_out = torch.empty_like(q) if q_out is None else q_out
    k_out = torch.empty_like(k) if k_out is None else k_out
    check(lib().jsm_rope_apply_qk(q.data_ptr(), q_out.data_ptr(), Hq, k.data_ptr(), k_out.data_ptr(), Hkv, dtype_of(q), table.data_ptr(), d,
                                  positions.data_ptr() if positions is not None else None, q.shape[0], stream_ptr()))
    return q_out, k_out


def attn_prefill(q, k, v, batch, Hq, Hkv, D, causal=True, scale=None, rope=None, impl=0, out=None):
    torch = _torch()
    out = torch.empty_like(q) if out is None else out
    Tq, Tk = q.shape[0] // batch, k.shape[0] // batch
    scale = float(D) ** -0.5 if scale is None else scale
    check(lib().jsm_attn_prefill(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dtype_of(q), batch, Tq, Tk,
                                 Hq, Hkv, D, int(causal), scale, rope.data_ptr() if rope is not None else None, impl,
                                 stream_ptr()))
    return out


def kv_append(pool, block_table, k, v, seq_ids, positions, Hkv, D, rope=None):
    T = k.shape[0]
    check(lib().jsm_kv_append(pool.data_ptr(), block_table.data_ptr(), block_table.shape[1], k.data_ptr(), v.data_ptr(),
                              k.stride(0), seq_ids.data_ptr(), positions.data_ptr(), T, Hkv, D,
                              rope.data_ptr() if rope is not None else None, stream_ptr()))


def attn_decode(q, pool, block_table, context_lens, Hq, Hkv, D, max_context, scale=None, rope=None, scratch=None,
                out=None):
    torch = _torch()
    n = q.shape[0]
    out = torch.empty(n, Hq * D, dtype=q.dtype, device=q.device) if out is None else out
    if scratch is None:
        nbytes = lib().jsm_attn_decode_scratch_bytes(n, Hq, D, max_context)
        scratch = torch.empty(nbytes // 4, dtype=torch.float32, device=q.device)
    scale = float(D) ** -0.5 if scale is None else scale
    check(lib().jsm_attn_decode(q.data_ptr(), q.stride(0), pool.data_ptr(), block_table.data_ptr(),
                                block_table.shape[1], context_lens.data_ptr(), n, Hq, Hkv, D, scale,
                                rope.data_ptr() if rope is not None else None, max_context, scratch.data_ptr(),
                                out.data_ptr(), stream_ptr()))
    return out


def attn_decode_append(q, k_new, v_new, pool, block_table, context_lens, Hq, Hkv, D, max_context, counters, scale=None,
                       rope=None, scratch=None, out=None):
    """jsm_attn_decode_append: append the new token of every sequence and attend, one launch."""
    torch = _torch()
    n = q.shape[0]
    out = torch.empty(n, Hq * D, dtype=q.dtype, device=q.device) if out is None else out
    if scratch is None:
        nbytes = lib().jsm_attn_decode_scratch_bytes(n, Hq, D, max_context)
        scratch = torch.empty(nbytes // 4, dtype=torch.float32, device=q.device)
    scale = float(D) ** -0.5 if scale is None else scale
    check(lib().jsm_attn_decode_append(q.data_ptr(), q.stride(0), k_new.data_ptr() if k_new is not None else None,
                                       v_new.data_ptr() if v_new is not None else None,
                                       k_new.stride(0) if k_new is not None else 0, pool.data_ptr(), block_table.data_ptr(),
                                       block_table.shape[1], context_lens.data_ptr(), n, Hq, Hkv, D, scale,
                                       rope.data_ptr() if rope is not None else None, max_context, scratch.data_ptr(),
                                       counters.data_ptr(), out.data_ptr(), stream_ptr()))
    return out


STATIC_SCRATCH_BYTES = 8 << 20


def attn_decode_static_scratch(q, pool, block_table, context_lens, Hq, Hkv, D, max_context, scale=None, rope=None,
                               out=None):
    """jsm_attn_decode_static_scratch: decode attention whose partials live in the library's built-in array
    (no allocation inside the call; `out` must be supplied by callers that may not allocate either)."""
    torch = _torch()
    n = q.shape[0]
    out = torch.empty(n, Hq * D, dtype=q.dtype, device=q.device) if out is None else out
    scale = float(D) ** -0.5 if scale is None else scale
    check(lib().jsm_attn_decode_static_scratch(q.data_ptr(), q.stride(0), pool.data_ptr(), block_table.data_ptr(),
                                               block_table.shape[1], context_lens.data_ptr(), n, Hq, Hkv, D, scale,
                                               rope.data_ptr() if rope is not None else None, max_context,
                                               out.data_ptr(), stream_ptr()))
    return out


def embedding(table, ids, pos_table=None, positions=None, out=None):
    torch = _torch()
    T, d = ids.shape[0], table.shape[1]
    out = torch.empty(T, d, dtype=table.dtype, device=table.device) if out is None else out
    check(lib().jsm_embedding(table.data_ptr(), pos_table.data_ptr() if pos_table is not None else None, ids.data_ptr(),
                              positions.data_ptr() if positions is not None else None, out.data_ptr(), dtype_of(table),
                              T, d, stream_ptr()))
    return out


def add_norm(kind, h, delta, gain, bias=None, eps=1e-5, h_out=None, y=None):
    torch = _torch()
    T, d = h.shape
    y = torch.empty_like(h) if y is None else y
    check(lib().jsm_add_norm(kind, h.data_ptr(), delta.data_ptr() if delta is not None else None,
                             h_out.data_ptr() if h_out is not None else None, y.data_ptr(), dtype_of(h),
                             gain.data_ptr() if gain is not None else None,
                             bias.data_ptr() if bias is not None else None, eps, T, d, stream_ptr()))
    return y


def fill(t, seed: int, tensor_id: int, dist: int, a: float, b: float):
    """Seeded fill of a contiguous tensor on its device (dist 0 normal(a,b), 1 uniform[a,b), 2 int[a,b))."""
    assert t.is_contiguous()
    if t.is_cuda:
        check(lib().jsm_fill(t.data_ptr(), dtype_of(t), t.numel(), seed, tensor_id, dist, a, b, stream_ptr()))
    else:
        check(lib().jsm_fill_host(t.data_ptr(), dtype_of(t), t.numel(), seed, tensor_id, dist, a, b))
    return t


def sample(logits, temperature=1.0, top_k=0, top_p=1.0, seed=0, step=0, out=None):
    """Tokens drawn from F32 logits [rows, vocab] (temperature, top-k, top-p); int32 [rows]."""
    torch = _torch()
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    check(lib().jsm_sample(logits.data_ptr(), logits.stride(0), rows, vocab, temperature, top_k, top_p, seed, step,
                           out.data_ptr(), stream_ptr()))
    return out


def check_device_errors():
    """Synchronise and raise JsmError(TIMEOUT) if a tensor-core kernel gave up on a wait since the last check."""
    check(lib().jsm_check_device_errors(stream_ptr()))


def launch_count() -> int:
    return int(lib().jsm_launch_count())
