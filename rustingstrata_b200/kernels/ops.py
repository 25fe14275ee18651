"""Python launchers of the CUDA kernels: torch tensors in, raw pointers out.

Every function launches on torch's current CUDA stream, checks what it can on the
host (devices, element types, shapes, contiguity, alignment) and raises on a bad
launch.  There is no CPU path and no library fallback: if the extension cannot be
built or loaded the first call raises :class:`~.build.KernelBuildError`.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_long, c_float, c_void_p
from typing import Optional

import torch

from ..dtypes import element_type
from .build import load_library

F32, BF16 = element_type("float32").code, element_type("bfloat16").code

STATUS_BAD_TOKEN = 1
STATUS_BAD_PAGE = 2
STATUS_WAIT_EXPIRED = 4
STATUS_NON_FINITE = 8
STATUS_BAD_PLAN = 16


class KernelError(RuntimeError):
    pass


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError(f"unsupported element type {t.dtype} (float32 and bfloat16 only)")
    return element_type(t.dtype).code


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _stream() -> c_void_p:
    """The stream to launch on.  Every launcher asks for it right before its launch, so this is also where a recorded
    chain of decode products (see :func:`begin_chain`) is sent off before any other kernel can overtake it."""
    flush_chain()
    return c_void_p(torch.cuda.current_stream().cuda_stream)


_LAUNCHES = 0


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for the decode-path kernels (default on); off gives plain stream order."""
    core().rs_core_set_pdl(1 if on else 0)
    bf16lib().rs_bf16_set_pdl(1 if on else 0)


def launch_count() -> int:
    """Kernels of this package launched so far by this process."""
    return _LAUNCHES


def _check(code: int, what: str, kernels: int = 1) -> None:
    global _LAUNCHES
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code}")
    _LAUNCHES += kernels


def _cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel launchers take CUDA tensors only; there is no CPU path")


def _rows_contiguous(t: torch.Tensor, name: str):
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be 2-D with unit stride along its last axis, got shape {tuple(t.shape)} "
                          f"strides {t.stride()}")


_core = None


def core():
    global _core
    if _core is None:
        lib = load_library("core")
        lib.rs_embed.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
        lib.rs_gather_i32.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        lib.rs_rmsnorm.argtypes = [c_void_p, c_long, c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_long,
                                   c_int, c_int, c_void_p]
        lib.rs_qk_norm_rope_kv.argtypes = [c_void_p, c_int, c_long, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                                           c_float, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                           c_int, c_int, c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_void_p]
        lib.rs_silu_mul.argtypes = [c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_void_p]
        lib.rs_residual_add.argtypes = [c_void_p, c_void_p, c_int, c_long, c_void_p]
        lib.rs_linear_simt.argtypes = [c_void_p, c_int, c_long, c_void_p, c_int, c_long, c_void_p, c_int, c_long,
                                       c_int, c_int, c_int, c_int, c_void_p]
        lib.rs_attention_simt.argtypes = [c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_int,
                                          c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                          c_int, c_float, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                          c_void_p]
        lib.rs_attention_simt_q_per_cta.argtypes = [c_int, c_int]
        lib.rs_attention_simt_partial_floats.argtypes = [c_int, c_int, c_int]
        lib.rs_attention_simt_partial_floats.restype = c_long
        lib.rs_fill_random.argtypes = [c_void_p, c_int, c_long, ctypes.c_ulonglong, c_long, c_void_p, c_float, c_float,
                                       c_void_p]
        lib.rs_sample.argtypes = [c_void_p, c_long, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
        _core = lib
    return _core


# ----------------------------------------------------------------------------- elementwise
def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> None:
    """out[t] = table[ids[t]] as float32.  ids int32 [T]; out float32 [T, H]."""
    _cuda(table, ids, out, status)
    T, H = out.shape
    if ids.dtype != torch.int32 or out.dtype != torch.float32 or not out.is_contiguous() or not table.is_contiguous():
        raise KernelError("embed: ids must be int32, out contiguous float32, table contiguous")
    if table.shape[1] != H or ids.numel() < T:
        raise KernelError(f"embed: table {tuple(table.shape)} / ids {ids.numel()} do not fit out {tuple(out.shape)}")
    _check(core().rs_embed(_ptr(table), dtype_code(table), _ptr(ids), _ptr(out), T, H, table.shape[0], _ptr(status),
                           _stream()), "embed")


def gather_i32(dst: torch.Tensor, src: torch.Tensor, idx: torch.Tensor, n: int) -> None:
    """dst[i] = src[idx[i]] for i < n, all int32 on the device (idx must point inside src)."""
    _cuda(dst, src, idx)
    if dst.dtype != torch.int32 or src.dtype != torch.int32 or idx.dtype != torch.int32 or dst.numel() < n or idx.numel() < n:
        raise KernelError("gather_i32: int32 tensors with at least n entries")
    _check(core().rs_gather_i32(_ptr(dst), _ptr(src), _ptr(idx), n, _stream()), "gather_i32")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None, pending=None) -> None:
    """out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * weight.  x float32 [*, n].

    ``pending``: a :class:`PendingSum` still owed to ``x``.  If it covers exactly the rows that are normed, one kernel
    adds the partial sums and norms the rows (the same bits as the two kernels in turn); else it is finished first."""
    _cuda(x, weight, out, rows)
    if _ACTIVE_CHAIN is not None and _ACTIVE_CHAIN.ops and pending is None and rows is None:
        nr = n_rows if n_rows is not None else x.shape[0]
        lib = bf16lib()
        if (nr <= lib.rs_decode_chain_max_rows() and x.dtype == torch.float32 and out.dtype == torch.bfloat16
                and x.dim() == 2 and out.dim() == 2 and x.stride(1) == 1 and out.stride(1) == 1
                and x.shape[1] == weight.numel() == out.shape[1] and x.shape[1] % 4 == 0
                and x.shape[1] <= lib.rs_decode_chain_max_norm_width() and x.stride(0) % 4 == 0 and out.stride(0) % 4 == 0
                and x.data_ptr() % 16 == 0 and out.data_ptr() % 8 == 0 and weight.data_ptr() % 16 == 0
                and weight.is_contiguous() and weight.dtype in (torch.float32, torch.bfloat16) and nr <= out.shape[0]):
            _ACTIVE_CHAIN.add_rmsnorm(x, weight, eps, out, nr)
            return
    if pending is not None and not pending.done:
        nr = n_rows if n_rows is not None else (out.shape[0] if rows is not None else x.shape[0])
        lib = bf16lib()
        if (rows is None and pending.out.data_ptr() == x.data_ptr() and pending.out.stride(0) == x.stride(0)
                and pending.n_rows == nr and pending.N == x.shape[1] == weight.numel() == out.shape[1]
                and x.dtype == torch.float32 and out.dtype == torch.bfloat16 and weight.is_contiguous()
                and weight.dtype in (torch.float32, torch.bfloat16) and nr <= out.shape[0] and x.stride(1) == 1 and out.stride(1) == 1
                and lib.rs_skinny_finish_rmsnorm_supported(_ptr(x), x.stride(0), pending.N, _ptr(weight), _ptr(out), out.stride(0))):
            pending.finish_with_rmsnorm(weight, eps, out)
            return
        pending.finish()
    _rows_contiguous(x, "rmsnorm x")
    _rows_contiguous(out, "rmsnorm out")
    n = x.shape[1]
    if x.dtype != torch.float32:
        raise KernelError("rmsnorm reads the float32 residual stream")
    if weight.numel() != n or out.shape[1] != n or not weight.is_contiguous():
        raise KernelError(f"rmsnorm: weight {tuple(weight.shape)} / out {tuple(out.shape)} do not fit width {n}")
    if n_rows is None:
        n_rows = out.shape[0] if rows is not None else x.shape[0]
    if n_rows > out.shape[0] or (rows is None and n_rows > x.shape[0]):
        raise KernelError("rmsnorm: more rows than the buffers hold")
    if rows is not None and (rows.dtype != torch.int32 or rows.numel() < n_rows):
        raise KernelError("rmsnorm: rows must be int32 with n_rows entries")
    _check(core().rs_rmsnorm(_ptr(x), x.stride(0), _ptr(rows), _ptr(weight), dtype_code(weight), float(eps),
                             _ptr(out), dtype_code(out), out.stride(0), n_rows, n, _stream()), "rmsnorm")


def qk_norm_rope_kv(qkv: torch.Tensor, n_tokens: int, n_q: int, n_kv: int, head_dim: int,
                    q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                    cos_sin: Optional[torch.Tensor], n_rot: int, positions: torch.Tensor, seq_of_token: torch.Tensor,
                    block_table: torch.Tensor, page_size: int, cache: torch.Tensor, write_kv: bool,
                    status: torch.Tensor, stream: int = 0) -> None:
    """Per-head norm and rotation of q (in place) and k, and the write of k and v into their pages.

    qkv: [T, (n_q + 2 n_kv) * head_dim] (only the q part when ``write_kv`` is false);
    cache: [pages, 2, n_kv, page_size, head_dim] of the same element type.
    positions: [T] or [T, n_streams] int32; column 0 is the token's place in the cache, column ``stream`` the
    position the rotation follows (a row of ``cos_sin``).
    """
    _cuda(qkv, q_weight, k_weight, cos_sin, positions, seq_of_token, block_table, cache, status)
    _rows_contiguous(qkv, "qkv")
    need = (n_q + (2 * n_kv if write_kv else 0)) * head_dim
    if qkv.shape[1] < need or qkv.shape[0] < n_tokens:
        raise KernelError(f"qk_norm_rope_kv: qkv {tuple(qkv.shape)} is smaller than {n_tokens} x {need}")
    if cache.dtype != qkv.dtype or not cache.is_contiguous():
        raise KernelError("qk_norm_rope_kv: cache must be contiguous and of the activations' element type")
    if tuple(cache.shape[1:]) != (2, n_kv, page_size, head_dim):
        raise KernelError(f"qk_norm_rope_kv: cache shape {tuple(cache.shape)} is not [pages, 2, {n_kv}, {page_size}, "
                          f"{head_dim}]")
    w_dt = F32
    for w in (q_weight, k_weight):
        if w is not None:
            if w.numel() != head_dim or not w.is_contiguous():
                raise KernelError("qk_norm_rope_kv: norm weights must hold head_dim values")
            w_dt = dtype_code(w)
    if q_weight is not None and k_weight is not None and q_weight.dtype != k_weight.dtype:
        raise KernelError("qk_norm_rope_kv: q and k norm weights must share an element type")
    if cos_sin is not None and (cos_sin.dtype != torch.float32 or cos_sin.shape[1] != n_rot or
                                not cos_sin.is_contiguous()):
        raise KernelError("qk_norm_rope_kv: cos_sin must be contiguous float32 [positions, n_rot]")
    for name, t in (("positions", positions), ("seq_of_token", seq_of_token), ("block_table", block_table)):
        if t.dtype != torch.int32:
            raise KernelError(f"qk_norm_rope_kv: {name} must be int32")
    n_streams = 1 if positions.dim() == 1 else positions.shape[1]
    if positions.dim() > 2 or not positions.is_contiguous() or positions.shape[0] < n_tokens or not 0 <= stream < n_streams:
        raise KernelError(f"qk_norm_rope_kv: positions must be contiguous [tokens] or [tokens, streams] and hold stream "
                          f"{stream}; got shape {tuple(positions.shape)}")
    _check(core().rs_qk_norm_rope_kv(
        _ptr(qkv), dtype_code(qkv), qkv.stride(0), n_q, n_kv, head_dim, _ptr(q_weight), _ptr(k_weight), w_dt,
        float(eps), _ptr(cos_sin), n_rot, 0 if cos_sin is None else cos_sin.shape[0], _ptr(positions), n_streams, stream,
        _ptr(seq_of_token), _ptr(block_table),
        block_table.stride(0), page_size, _ptr(cache), cache.stride(0), cache.shape[0], 1 if write_kv else 0,
        n_tokens, _ptr(status), _stream()), "qk_norm_rope_kv")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, n_rows: int) -> None:
    """out[r, c] = silu(gate_up[r, c]) * gate_up[r, I + c], I = out.shape[1]."""
    _cuda(gate_up, out)
    _rows_contiguous(gate_up, "gate_up")
    _rows_contiguous(out, "out")
    I = out.shape[1]
    if gate_up.shape[1] != 2 * I or gate_up.dtype != out.dtype or n_rows > min(gate_up.shape[0], out.shape[0]):
        raise KernelError(f"silu_mul: gate_up {tuple(gate_up.shape)} does not fit out {tuple(out.shape)}")
    _check(core().rs_silu_mul(_ptr(gate_up), gate_up.stride(0), _ptr(out), out.stride(0), dtype_code(out), n_rows, I,
                              _stream()), "silu_mul")


def residual_add(x: torch.Tensor, delta: torch.Tensor, n_rows: int) -> None:
    """x[:n_rows] += delta[:n_rows] in float32 (both contiguous, same width)."""
    _cuda(x, delta)
    if x.dtype != torch.float32 or not x.is_contiguous() or not delta.is_contiguous() or x.shape[1] != delta.shape[1]:
        raise KernelError("residual_add: x must be contiguous float32 and delta contiguous of the same width")
    _check(core().rs_residual_add(_ptr(x), _ptr(delta), dtype_code(delta), n_rows * x.shape[1], _stream()),
           "residual_add")


def fill_random(out: torch.Tensor, key: int, table: Optional[torch.Tensor], scale: float, shift: float,
                first: int = 0) -> None:
    """out.flatten()[i] = shift + scale * table[z_i >> 48] with z_i the 64-bit hash of (key, first + i): the device
    half of the random-weights generator (weights/random_init.py is the host half and gives the same bits).
    ``out`` float32 or bfloat16; int32 takes the low bit of z_i and needs no table."""
    _cuda(out, table)
    if not out.is_contiguous():
        raise KernelError("fill_random: out must be contiguous")
    if out.dtype == torch.int32:
        code = element_type("int32").code
    else:
        code = dtype_code(out)
        if table is None or table.dtype != torch.float32 or table.numel() != 1 << 16 or not table.is_contiguous():
            raise KernelError("fill_random: table must be the 65,536 float32 normal quantiles")
    _check(core().rs_fill_random(_ptr(out), code, out.numel(), key & 0xFFFFFFFFFFFFFFFF, first, _ptr(table), float(scale),
                                 float(shift), _stream()), "fill_random")


# ----------------------------------------------------------------------------- matrix products
def linear_simt(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, n_rows: int, accumulate: bool = False) -> None:
    """out[:n_rows] (=|+=) a[:n_rows] @ weight.T on CUDA cores, float32 accumulation."""
    _cuda(a, weight, out)
    _rows_contiguous(a, "a")
    _rows_contiguous(weight, "weight")
    _rows_contiguous(out, "out")
    N, K = weight.shape
    if a.shape[1] != K or out.shape[1] != N or n_rows > min(a.shape[0], out.shape[0]):
        raise KernelError(f"linear: a {tuple(a.shape)} x weight {tuple(weight.shape)} -> out {tuple(out.shape)} "
                          f"for {n_rows} rows does not fit")
    _check(core().rs_linear_simt(_ptr(a), dtype_code(a), a.stride(0), _ptr(weight), dtype_code(weight),
                                 weight.stride(0), _ptr(out), dtype_code(out), out.stride(0), n_rows, N, K,
                                 1 if accumulate else 0, _stream()), "linear_simt")


_bf16 = None


def bf16lib():
    global _bf16
    if _bf16 is None:
        lib = load_library("bf16")
        lib.rs_gemm_bf16_tc.argtypes = [c_void_p, c_long, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int,
                                        c_int, c_int, c_int, c_void_p, c_void_p]
        lib.rs_skinny_gemm_bf16.argtypes = [c_void_p, c_long, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int,
                                            c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]
        lib.rs_skinny_gemm_workspace_floats.restype = c_long
        lib.rs_skinny_finish.argtypes = [c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_int, c_void_p]
        lib.rs_skinny_finish_rmsnorm_supported.argtypes = [c_void_p, c_long, c_int, c_void_p, c_void_p, c_long]
        lib.rs_skinny_finish_rmsnorm.argtypes = [c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int,
                                                 c_float, c_void_p, c_long, c_void_p]
        lib.rs_decode_chain.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
        lib.rs_mid_gemm_bf16.argtypes = [c_void_p, c_long, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int,
                                         c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]
        lib.rs_mid_finish.argtypes = lib.rs_skinny_finish.argtypes
        lib.rs_mid_finish_rmsnorm.argtypes = lib.rs_skinny_finish_rmsnorm.argtypes
        lib.rs_mid_gemm_workspace_floats.restype = c_long
        lib.rs_attention_decode_bf16.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int,
                                                 c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                 c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                 c_void_p, c_void_p]
        lib.rs_attention_decode_build_items.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
        lib.rs_attention_decode_bf16_supported.argtypes = [c_int, c_int, c_int, c_int]
        lib.rs_attention_prefill_bf16.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int,
                                                  c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                  c_int, c_int, c_float, c_void_p, c_void_p]
        lib.rs_attention_prefill_tc.argtypes = [c_void_p, c_long, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int,
                                                c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                c_int, c_float, c_void_p, c_void_p]
        lib.rs_attention_prefill_tc_supported.argtypes = [c_int, c_int, c_int, c_int]
        lib.rs_attention_prefill_tc_q_per_cta.argtypes = [c_int, c_int]
        lib.rs_attention_prefill_bf16_supported.argtypes = [c_int, c_int, c_int]
        lib.rs_attention_prefill_bf16_q_per_cta.argtypes = [c_int, c_int]
        _bf16 = lib
    return _bf16


EPI_STORE_BF16, EPI_STORE_F32, EPI_ADD_F32, EPI_SWIGLU_BF16 = 0, 1, 2, 3


def tensor_core_shape_ok(a: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the bfloat16 tensor-core kernels take this product: both operands bfloat16, every row
    16-byte aligned (K and the row pitches multiples of 8 elements, base pointers multiples of 16)."""
    if a.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        return False
    K = weight.shape[1]
    return (K % 8 == 0 and a.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0
            and weight.data_ptr() % 16 == 0)


def _epilogue_code(out: torch.Tensor, accumulate: bool, swiglu: bool) -> int:
    if swiglu:
        if out.dtype != torch.bfloat16 or accumulate:
            raise KernelError("the fused SiLU(gate)*up epilogue writes bfloat16 and does not accumulate")
        return EPI_SWIGLU_BF16
    if out.dtype == torch.bfloat16:
        if accumulate:
            raise KernelError("accumulating products go into the float32 residual stream")
        return EPI_STORE_BF16
    if out.dtype == torch.float32:
        return EPI_ADD_F32 if accumulate else EPI_STORE_F32
    raise KernelError(f"unsupported output element type {out.dtype}")


def _check_product(a, weight, out, n_rows, swiglu):
    _cuda(a, weight, out)
    _rows_contiguous(a, "a")
    _rows_contiguous(weight, "weight")
    _rows_contiguous(out, "out")
    N, K = weight.shape
    n_out = N // 2 if swiglu else N
    if a.shape[1] != K or out.shape[1] != n_out or n_rows > min(a.shape[0], out.shape[0]) or (swiglu and N % 2):
        raise KernelError(f"linear: a {tuple(a.shape)} x weight {tuple(weight.shape)} -> out {tuple(out.shape)} "
                          f"for {n_rows} rows does not fit")
    return N, K


def gemm_bf16_tc(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, n_rows: int, accumulate: bool = False,
                 swiglu: bool = False, status: Optional[torch.Tensor] = None, bn: int = 0, max_ctas: int = 0) -> None:
    """out[:n_rows] (=|+=) a[:n_rows] @ weight.T on the tcgen05 tensor cores (csrc/gemm_tcgen05.cu).
    ``swiglu``: weight rows alternate gate, up and out[:, j] = silu(gate_j) * up_j."""
    N, K = _check_product(a, weight, out, n_rows, swiglu)
    if not tensor_core_shape_ok(a, weight):
        raise KernelError(f"gemm_bf16_tc refuses a {tuple(a.shape)} {a.dtype} stride {a.stride(0)} x weight "
                          f"{tuple(weight.shape)} {weight.dtype}: rows must be bfloat16 and 16-byte aligned")
    if status is None:
        status = _default_status(a.device)
    _check(bf16lib().rs_gemm_bf16_tc(_ptr(a), a.stride(0), a.shape[0], _ptr(weight), weight.stride(0), _ptr(out),
                                     out.stride(0), n_rows, N, K, _epilogue_code(out, accumulate, swiglu), bn, max_ctas,
                                     _ptr(status), _stream()), "gemm_bf16_tc")


SKINNY_MAX_ROWS = 64     # what the kernel takes
SKINNY_MAX_WEIGHT = 1 << 28   # weights of this many elements or more (an output head) stream faster through the tcgen05 kernel
SKINNY_ROWS = 8          # up to here the engine prefers it; from 9 rows the stream-K tcgen05 kernel is as fast or faster
_SKINNY_SCRATCH = {}


def _skinny_scratch(device):
    """Workspace of the skinny product (partials of shared row tiles), one per device, made at the first call
    (before any graph capture: the engine runs every shape once eagerly first)."""
    ws = _SKINNY_SCRATCH.get(device)
    if ws is None:
        ws = _SKINNY_SCRATCH[device] = torch.empty(int(bf16lib().rs_skinny_gemm_workspace_floats()), dtype=torch.float32,
                                                   device=device)
    return ws


class PendingSum:
    """A product into the float32 residual stream whose last step is still owed: the partial sums of the weight tiles
    that several CTAs shared lie in the product's workspace and have not been added to ``out`` yet.  Whoever reads
    ``out`` next either takes the object along (``rmsnorm(..., pending=...)`` adds the partials while it reads the
    rows) or calls :meth:`finish` first.  No other product of the same kind may run in between: it would overwrite the
    workspace.  ``kind``: "skinny" (up to 8 rows) or "mid" (the stream-K tcgen05 product, up to 128 rows)."""

    def __init__(self, kind: str, out: torch.Tensor, n_rows: int, N: int, K: int, workspace: torch.Tensor, max_ctas: int):
        self.kind, self.out, self.n_rows, self.N, self.K = kind, out, n_rows, N, K
        self.workspace, self.max_ctas = workspace, max_ctas
        self.done = False

    def finish(self) -> None:
        """out += the partial sums (the small kernel that the product would have launched itself)."""
        if not self.done:
            self.done = True
            fn = bf16lib().rs_skinny_finish if self.kind == "skinny" else bf16lib().rs_mid_finish
            _check(fn(_ptr(self.out), self.out.stride(0), self.n_rows, self.N, self.K, _ptr(self.workspace), self.max_ctas,
                      _stream()), self.kind + "_finish")

    def finish_with_rmsnorm(self, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
        """The same and out[r] = RMSNorm(self.out[r]) * weight, in one kernel."""
        self.done = True
        fn = bf16lib().rs_skinny_finish_rmsnorm if self.kind == "skinny" else bf16lib().rs_mid_finish_rmsnorm
        _check(fn(_ptr(self.out), self.out.stride(0), self.n_rows, self.N, self.K, _ptr(self.workspace), self.max_ctas,
                  _ptr(weight), dtype_code(weight), float(eps), _ptr(out), out.stride(0), _stream()),
               self.kind + "_finish_rmsnorm")


SKINNY_DEFER_ROWS = 8    # the deferred form exists for the thread layout of up to 8 rows
DEFER_SUMS = True        # whether linear() lets a product leave its last sum to the next reader when the caller allows it


def skinny_gemm_bf16(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, n_rows: int, accumulate: bool = False,
                     swiglu: bool = False, status: Optional[torch.Tensor] = None, max_ctas: int = 0,
                     defer: bool = False) -> Optional[PendingSum]:
    """out[:n_rows] (=|+=) a[:n_rows] @ weight.T for n_rows <= 64: persistent CTAs stream the weight through a
    TMA-fed ring of shared-memory stages (csrc/skinny_gemm_tma.cu).  With ``defer`` (float32 +=, up to 8 rows) the
    kernel that adds up the shared tiles is not launched and a :class:`PendingSum` is returned instead."""
    N, K = _check_product(a, weight, out, n_rows, swiglu)
    if defer and not (accumulate and out.dtype == torch.float32 and n_rows <= SKINNY_DEFER_ROWS):
        raise KernelError("skinny_gemm_bf16 defers only a float32 += of up to 8 rows")
    if n_rows > SKINNY_MAX_ROWS or not tensor_core_shape_ok(a, weight) or N <= 0:
        raise KernelError(f"skinny_gemm_bf16 refuses {n_rows} rows of a {tuple(a.shape)} {a.dtype} x weight "
                          f"{tuple(weight.shape)} {weight.dtype}: at most {SKINNY_MAX_ROWS} rows, bfloat16, 16-byte aligned")
    if status is None:
        status = _default_status(a.device)
    ws = _skinny_scratch(a.device)
    _check(bf16lib().rs_skinny_gemm_bf16(_ptr(a), a.stride(0), a.shape[0], _ptr(weight), weight.stride(0), _ptr(out),
                                         out.stride(0), n_rows, N, K, _epilogue_code(out, accumulate, swiglu), _ptr(ws),
                                         max_ctas, 1 if defer else 0, _ptr(status), _stream()), "skinny_gemm_bf16", 1 if defer else 2)
    return PendingSum("skinny", out, n_rows, N, K, ws, max_ctas) if defer else None


MID_MAX_ROWS = 128       # what the stream-K tcgen05 kernel takes; the engine uses it from SKINNY_ROWS + 1 rows up to here
_MID_SCRATCH = {}


def _mid_scratch(device):
    """Workspace of the stream-K tcgen05 product, one per device, made at the first call."""
    ws = _MID_SCRATCH.get(device)
    if ws is None:
        ws = _MID_SCRATCH[device] = torch.empty(int(bf16lib().rs_mid_gemm_workspace_floats()), dtype=torch.float32,
                                                device=device)
    return ws


def mid_gemm_bf16(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, n_rows: int, accumulate: bool = False,
                  swiglu: bool = False, status: Optional[torch.Tensor] = None, max_ctas: int = 0,
                  defer: bool = False) -> Optional[PendingSum]:
    """out[:n_rows] (=|+=) a[:n_rows] @ weight.T for n_rows <= 128 on the tensor cores with the operands swapped
    (rows of the weight fill the 128-row side of the MMA) and the work dealt to the SMs in equal shares of k
    (csrc/mid_gemm_tcgen05.cu).  With ``defer`` (float32 += only) the kernel that adds up the shared tiles is not
    launched and a :class:`PendingSum` is returned instead."""
    N, K = _check_product(a, weight, out, n_rows, swiglu)
    if defer and not (accumulate and out.dtype == torch.float32):
        raise KernelError("mid_gemm_bf16 defers only a float32 +=")
    if n_rows > MID_MAX_ROWS or not tensor_core_shape_ok(a, weight):
        raise KernelError(f"mid_gemm_bf16 refuses {n_rows} rows of a {tuple(a.shape)} {a.dtype} x weight "
                          f"{tuple(weight.shape)} {weight.dtype}: at most {MID_MAX_ROWS} rows, bfloat16, 16-byte aligned")
    if status is None:
        status = _default_status(a.device)
    ws = _mid_scratch(a.device)
    _check(bf16lib().rs_mid_gemm_bf16(_ptr(a), a.stride(0), a.shape[0], _ptr(weight), weight.stride(0), _ptr(out),
                                      out.stride(0), n_rows, N, K, _epilogue_code(out, accumulate, swiglu), _ptr(ws),
                                      max_ctas, 1 if defer else 0, _ptr(status), _stream()), "mid_gemm_bf16",
           1 if defer else 2)
    return PendingSum("mid", out, n_rows, N, K, ws, max_ctas) if defer else None


_STATUS = {}


def _default_status(device) -> torch.Tensor:
    t = _STATUS.get(device)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _STATUS[device] = t
    return t


# ----------------------------------------------------------------------------- a chain of decode products in one kernel
class RsChainOp(ctypes.Structure):
    """One operation of a chain, as csrc/decode_chain.cu takes it."""
    _fields_ = [("type", c_int), ("M", c_int), ("N", c_int), ("K", c_int), ("epi", c_int), ("owed", c_int), ("w_dt", c_int),
                ("reserved", c_int), ("lda", c_long), ("a_rows", c_long), ("ldw", c_long), ("ldc", c_long), ("out_stride", c_long),
                ("A", c_void_p), ("W", c_void_p), ("C", c_void_p), ("w", c_void_p), ("out", c_void_p), ("eps", c_float),
                ("reserved2", c_int)]


CHAIN_GEMV, CHAIN_REDUCE, CHAIN_ROWNORM = 0, 1, 2
CHAIN_DECODE = False     # whether the engine chains the products of a decode step of up to 8 tokens (begin_chain); measured
                         # slower than the separate kernels under programmatic dependent launch, so it is off
_CHAIN_BUFFERS = {}


class _Chain:
    """The products of up to 8 rows, and the row norms between them, that have been asked for since the last kernel of
    another kind: they wait here and leave as ONE persistent kernel (csrc/decode_chain.cu) when anything else is about
    to be launched, so that the weights of a whole run of dependent products stream without a kernel boundary."""

    def __init__(self, status: torch.Tensor):
        self.status = status
        self.ops = []            # RsChainOp
        self.keep = []           # the tensors the operations point into
        self.n_products = 0
        self.open_product = None   # the last op, if it is a product whose shared tiles nobody has been told to finish
        self.launches = 0

    def _room(self, n_ops: int, n_products: int = 0) -> None:
        lib = bf16lib()
        if (len(self.ops) + n_ops > lib.rs_decode_chain_max_ops()
                or self.n_products + n_products > lib.rs_decode_chain_max_products()):
            self.flush()

    def _close_product(self) -> None:
        """The product recorded last leaves its shared tiles to a REDUCE operation (nobody else took them)."""
        g = self.open_product
        if g is not None:
            self.open_product = None
            r = RsChainOp.from_buffer_copy(g)
            r.type = CHAIN_REDUCE
            self.ops.append(r)

    def add_product(self, a, weight, out, n_rows, epi) -> None:
        self._close_product()
        self._room(2, 1)
        N, K = weight.shape
        op = RsChainOp(type=CHAIN_GEMV, M=n_rows, N=N, K=K, epi=epi, lda=a.stride(0), a_rows=a.shape[0], ldw=weight.stride(0),
                       ldc=out.stride(0), A=a.data_ptr(), W=weight.data_ptr(), C=out.data_ptr())
        self.ops.append(op)
        self.keep += [a, weight, out]
        self.n_products += 1
        self.open_product = op

    def add_rmsnorm(self, x, weight, eps, out, n_rows) -> None:
        g = self.open_product
        owed = (g is not None and g.epi == EPI_ADD_F32 and g.C == x.data_ptr() and g.ldc == x.stride(0) and g.M == n_rows
                and g.N == x.shape[1])
        if owed:
            self.open_product = None                 # the norm adds the product's partial sums while it reads the rows
        else:
            self._close_product()
        self._room(1)
        self.ops.append(RsChainOp(type=CHAIN_ROWNORM, M=n_rows, N=x.shape[1], K=g.K if owed else 1, owed=1 if owed else 0,
                                  w_dt=dtype_code(weight), ldc=x.stride(0), out_stride=out.stride(0), C=x.data_ptr(),
                                  w=weight.data_ptr(), out=out.data_ptr(), eps=float(eps)))
        self.keep += [x, weight, out]

    def flush(self) -> None:
        if not self.ops:
            return
        self._close_product()
        ops, self.ops, keep, self.keep = self.ops, [], self.keep, []
        self.n_products = 0
        arr = (RsChainOp * len(ops))(*ops)
        dev = self.status.device
        bufs = _CHAIN_BUFFERS.get(dev)
        if bufs is None:
            bufs = _CHAIN_BUFFERS[dev] = torch.zeros(2, dtype=torch.int32, device=dev)
        ws = _skinny_scratch(dev)
        global _FLUSHING
        _FLUSHING = True
        try:
            stream = c_void_p(torch.cuda.current_stream().cuda_stream)
            _check(bf16lib().rs_decode_chain(ctypes.cast(arr, c_void_p), len(ops), _ptr(ws), _ptr(bufs), _ptr(self.status), stream),
                   "decode_chain")
        finally:
            _FLUSHING = False
        self.launches += 1
        del keep


_ACTIVE_CHAIN: Optional[_Chain] = None
_FLUSHING = False


def chain_max_rows() -> int:
    return int(bf16lib().rs_decode_chain_max_rows())


def begin_chain(status: torch.Tensor) -> None:
    """From here to :func:`end_chain`, products of up to 8 bfloat16 rows (``linear``, ``linear_swiglu``) and the row
    norms between them are recorded instead of launched, and leave as one kernel when any other kernel of this module is
    asked for or the chain is ended.  Only for callers that touch the tensors involved through this module alone in
    between (torch operations on them would not see the recorded work)."""
    global _ACTIVE_CHAIN
    if _ACTIVE_CHAIN is not None:
        raise KernelError("a chain of decode products is already being recorded")
    _ACTIVE_CHAIN = _Chain(status)


def end_chain() -> int:
    """Launches what is recorded and stops recording; returns the number of chain kernels launched since begin_chain."""
    global _ACTIVE_CHAIN
    ch, _ACTIVE_CHAIN = _ACTIVE_CHAIN, None
    if ch is None:
        return 0
    ch.flush()
    return ch.launches


def flush_chain() -> None:
    if _ACTIVE_CHAIN is not None and not _FLUSHING:
        _ACTIVE_CHAIN.flush()


def reset_chain_barrier() -> None:
    """After a chain kernel gave up on a wait its arrival counter may be left mid-count: set it back."""
    for t in _CHAIN_BUFFERS.values():
        t.zero_()


def _chain_takes_product(a, weight, out, n_rows, swiglu: bool) -> bool:
    if _ACTIVE_CHAIN is None:            # asked first: the 32-bit engine must not load (or compile) the bfloat16 library
        return False
    lib = bf16lib()
    return (n_rows <= lib.rs_decode_chain_max_rows() and tensor_core_shape_ok(a, weight)
            and weight.numel() < SKINNY_MAX_WEIGHT and out.dtype in (torch.bfloat16, torch.float32)
            and a.is_cuda and weight.is_cuda and out.is_cuda)


def linear(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, n_rows: int, accumulate: bool = False,
           status: Optional[torch.Tensor] = None, may_defer: bool = False) -> Optional[PendingSum]:
    """The engine's matrix product: the tensor-core kernels for bfloat16 operands whose rows are 16-byte
    aligned (skinny kernel up to 8 rows, stream-K tcgen05 kernel up to 128, tiled tcgen05 kernel above), the
    CUDA-core kernel for everything else
    (the 32-bit engine, float32-stored weights, odd widths).  ``may_defer``: the caller hands a :class:`PendingSum`
    on to the next reader of ``out`` if the kernel that runs can leave one (else None comes back and ``out`` is whole)."""
    if _chain_takes_product(a, weight, out, n_rows, False):
        _check_product(a, weight, out, n_rows, False)
        _ACTIVE_CHAIN.add_product(a, weight, out, n_rows, _epilogue_code(out, accumulate, False))
        return None
    if tensor_core_shape_ok(a, weight) and out.dtype in (torch.bfloat16, torch.float32):
        if n_rows <= SKINNY_ROWS and weight.numel() < SKINNY_MAX_WEIGHT:
            defer = may_defer and DEFER_SUMS and accumulate and out.dtype == torch.float32 and n_rows <= SKINNY_DEFER_ROWS
            return skinny_gemm_bf16(a, weight, out, n_rows, accumulate, status=status, defer=defer)
        elif n_rows <= MID_MAX_ROWS:
            return mid_gemm_bf16(a, weight, out, n_rows, accumulate, status=status,
                                 defer=may_defer and DEFER_SUMS and accumulate and out.dtype == torch.float32)
        else:
            gemm_bf16_tc(a, weight, out, n_rows, accumulate, status=status)
    else:
        linear_simt(a, weight, out, n_rows, accumulate)


def linear_swiglu(a: torch.Tensor, weight_interleaved: torch.Tensor, out: torch.Tensor, n_rows: int,
                  status: Optional[torch.Tensor] = None) -> None:
    """out[:, j] = silu(a @ w[2j]) * (a @ w[2j+1]) in one kernel; only for shapes ``tensor_core_shape_ok`` takes."""
    if _chain_takes_product(a, weight_interleaved, out, n_rows, True):
        _check_product(a, weight_interleaved, out, n_rows, True)
        _ACTIVE_CHAIN.add_product(a, weight_interleaved, out, n_rows, _epilogue_code(out, False, True))
        return
    if n_rows <= SKINNY_ROWS:
        skinny_gemm_bf16(a, weight_interleaved, out, n_rows, swiglu=True, status=status)
    elif n_rows <= MID_MAX_ROWS:
        mid_gemm_bf16(a, weight_interleaved, out, n_rows, swiglu=True, status=status)
    else:
        gemm_bf16_tc(a, weight_interleaved, out, n_rows, swiglu=True, status=status)


# ----------------------------------------------------------------------------- attention
def attention_q_per_cta(n_q: int, n_kv: int) -> int:
    return int(core().rs_attention_simt_q_per_cta(n_q, n_kv))


def attention_partial_floats(total_splits: int, n_q: int, head_dim: int) -> int:
    return int(core().rs_attention_simt_partial_floats(total_splits, n_q, head_dim))


def attention_simt(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                   q_start: torch.Tensor, kv_len: torch.Tensor, work: torch.Tensor, n_work: int, n_q: int, n_kv: int,
                   head_dim: int, page_size: int, window: int, scale: float, decode: bool, status: torch.Tensor,
                   split_keys: int = 128, max_splits: int = 1, split_start: Optional[torch.Tensor] = None,
                   total_splits: int = 0, partial: Optional[torch.Tensor] = None,
                   slopes: Optional[torch.Tensor] = None) -> None:
    """Paged causal attention (see csrc/attention_simt.cu).  q/out: [T, >= n_q*head_dim] views.

    ``slopes``: float32 [n_q] or None: slopes[h] * (key position - query position) is added to every scaled score of
    head h (a position encoding that biases scores by distance instead of rotating q and k).

    Decode form: ``partial`` is the workspace of un-normalised partial results, one slot of n_q * (head_dim + 2)
    float32 values per (sequence, split); ``split_start[w]`` is the first slot of sequence w and ``total_splits`` the
    slots the caller knows the step uses (0 when it cannot say, as for a captured step whose lengths change from
    replay to replay).  The kernels are told how many slots the workspace holds and flag a slot beyond it
    (STATUS_BAD_PLAN) instead of writing there."""
    _cuda(q, out, cache, block_table, q_start, kv_len, work, status, partial, split_start)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if q.dtype != cache.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q, out and cache must share an element type")
    if tuple(cache.shape[1:]) != (2, n_kv, page_size, head_dim) or not cache.is_contiguous():
        raise KernelError(f"attention: cache shape {tuple(cache.shape)} is not [pages, 2, {n_kv}, {page_size}, {head_dim}]")
    if head_dim % 16 or head_dim > 256:
        raise KernelError(f"attention: head size {head_dim} is not a multiple of 16 up to 256")
    if n_q % n_kv:
        raise KernelError(f"attention: {n_q} query heads are not a multiple of {n_kv} key/value heads")
    for name, t in (("block_table", block_table), ("q_start", q_start), ("kv_len", kv_len), ("work", work)):
        if t.dtype != torch.int32:
            raise KernelError(f"attention: {name} must be int32")
    if slopes is not None and (slopes.dtype != torch.float32 or slopes.numel() != n_q or not slopes.is_contiguous() or not slopes.is_cuda):
        raise KernelError(f"attention: slopes must be contiguous float32 [{n_q}] on the device")
    slots = 0
    if decode:
        if split_start is None or split_start.dtype != torch.int32:
            raise KernelError("attention: the decode form needs int32 split_start")
        slots = _partial_slots(partial, total_splits, n_q, head_dim, "attention")
    _check(core().rs_attention_simt(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), dtype_code(q), _ptr(cache), cache.stride(0), cache.shape[0],
        page_size, _ptr(block_table), block_table.stride(0), _ptr(q_start), _ptr(kv_len), _ptr(work), n_work, n_q,
        n_kv, head_dim, int(window), float(scale), 1 if decode else 0, split_keys, max_splits, _ptr(split_start),
        _ptr(partial), slots, _ptr(slopes),
        _ptr(status), _stream()), "attention_simt", 2 if decode else 1)


def _partial_slots(partial: Optional[torch.Tensor], total_splits: int, n_q: int, head_dim: int, who: str) -> int:
    """Slots of partial results the workspace holds; raises if the step is known to need more."""
    if partial is None or partial.dtype != torch.float32 or not partial.is_contiguous():
        raise KernelError(f"{who}: the decode form needs a contiguous float32 workspace of partial results")
    slots = min(partial.numel() // (n_q * (head_dim + 2)), 0x7FFFFFFF)
    if slots < max(1, total_splits):
        raise KernelError(f"{who}: the step's {max(1, total_splits)} (sequence, split) pairs need "
                          f"{attention_partial_floats(max(1, total_splits), n_q, head_dim)} float32 values of partial "
                          f"workspace, {partial.numel()} were given")
    return int(slots)


def attention_prefill_kernel(dtype: torch.dtype, n_q: int, n_kv: int, head_dim: int, page_size: int, force: str = "") -> str:
    """Which kernel ``attention_prefill`` runs for this shape: "tc" (tcgen05, head 64/128, page size a power of
    two from 8 to 128), "mma" (mma.sync, head 32/64/96/128) or "simt" (everything else, and float32)."""
    if force:
        return force
    if dtype == torch.bfloat16:
        if bf16lib().rs_attention_prefill_tc_supported(n_q, n_kv, head_dim, page_size):
            return "tc"
        if bf16lib().rs_attention_prefill_bf16_supported(n_q, n_kv, head_dim):
            return "mma"
    return "simt"


def attention_prefill_fast_ok(dtype: torch.dtype, n_q: int, n_kv: int, head_dim: int) -> bool:
    """Whether a tensor-core portion kernel takes this shape (bfloat16, head size 32/64/96/128)."""
    return dtype == torch.bfloat16 and bool(bf16lib().rs_attention_prefill_bf16_supported(n_q, n_kv, head_dim))


def attention_prefill_q_per_cta(dtype: torch.dtype, n_q: int, n_kv: int, head_dim: int, page_size: int = 16,
                                force: str = "") -> int:
    """Query tokens per work item of the portion form, for the kernel ``attention_prefill`` will pick."""
    kind = attention_prefill_kernel(dtype, n_q, n_kv, head_dim, page_size, force)
    if kind == "tc":
        return int(bf16lib().rs_attention_prefill_tc_q_per_cta(n_q, n_kv))
    if kind == "mma":
        return int(bf16lib().rs_attention_prefill_bf16_q_per_cta(n_q, n_kv))
    return attention_q_per_cta(n_q, n_kv)


def attention_prefill(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                      q_start: torch.Tensor, kv_len: torch.Tensor, work: torch.Tensor, n_work: int, n_q: int, n_kv: int,
                      head_dim: int, page_size: int, window: int, scale: float, status: torch.Tensor,
                      force: str = "", slopes: Optional[torch.Tensor] = None) -> None:
    """Attention of prompt portions; ``work`` lists (sequence, first query) tiles of ``attention_prefill_q_per_cta``
    tokens.  tcgen05 kernel (csrc/attention_prefill_tc.cu), mma.sync kernel (csrc/attention_prefill_mma.cu) or
    CUDA cores, whichever takes the shape; ``force`` names one.  Score biases (``slopes``) are the CUDA-core kernel's."""
    kind = attention_prefill_kernel(q.dtype, n_q, n_kv, head_dim, page_size, force)
    if slopes is not None and kind != "simt":
        raise KernelError("attention_prefill: only the CUDA-core kernel (force='simt') adds score biases")
    if kind == "simt":
        attention_simt(q, out, cache, block_table, q_start, kv_len, work, n_work, n_q, n_kv, head_dim, page_size, window,
                       scale, False, status, slopes=slopes)
        return
    _cuda(q, out, cache, block_table, q_start, kv_len, work, status)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or q.dtype != torch.bfloat16 or not cache.is_contiguous():
        raise KernelError("attention_prefill: q, out and cache must be bfloat16 and the cache contiguous")
    if tuple(cache.shape[1:]) != (2, n_kv, page_size, head_dim):
        raise KernelError(f"attention_prefill: cache shape {tuple(cache.shape)} is not [pages, 2, {n_kv}, {page_size}, {head_dim}]")
    for name, t in (("block_table", block_table), ("q_start", q_start), ("kv_len", kv_len), ("work", work)):
        if t.dtype != torch.int32:
            raise KernelError(f"attention_prefill: {name} must be int32")
    if kind == "tc":
        fn = bf16lib().rs_attention_prefill_tc
        _check(fn(
            _ptr(q), q.stride(0), min(q.shape[0], out.shape[0]), _ptr(out), out.stride(0), _ptr(cache), cache.stride(0), cache.shape[0],
            page_size, _ptr(block_table), block_table.stride(0), _ptr(q_start), _ptr(kv_len), _ptr(work), n_work, n_q, n_kv,
            head_dim, int(window), float(scale), _ptr(status), _stream()), "attention_prefill_" + kind)
        return
    _check(bf16lib().rs_attention_prefill_bf16(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cache), cache.stride(0), cache.shape[0], page_size,
        _ptr(block_table), block_table.stride(0), _ptr(q_start), _ptr(kv_len), _ptr(work), n_work, n_q, n_kv, head_dim,
        int(window), float(scale), _ptr(status), _stream()), "attention_prefill_bf16")


def attention_decode_fast_ok(dtype: torch.dtype, n_q: int, n_kv: int, head_dim: int, page_size: int = 16) -> bool:
    """Whether the tensor-core decode kernel takes this shape (bfloat16, head size 64 or 128, group <= 16, pages of
    8 to 128 tokens, a power of two)."""
    return dtype == torch.bfloat16 and bool(
        bf16lib().rs_attention_decode_bf16_supported(n_q, n_kv, head_dim, page_size))


def attention_decode_loads_per_page() -> int:
    """TMA loads the tensor-core decode kernel issued per page of an item in its most recent launch: 1 when the
    driver took the 5-d map of the cache, else one per K/V and 64-wide half of the head."""
    return int(bf16lib().rs_attention_decode_bf16_loads_per_page())


def attention_decode(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                     q_start: torch.Tensor, kv_len: torch.Tensor, work: torch.Tensor, n_work: int, n_q: int, n_kv: int,
                     head_dim: int, page_size: int, window: int, scale: float, status: torch.Tensor, split_keys: int,
                     max_splits: int, split_start: torch.Tensor, total_splits: int, partial: torch.Tensor,
                     force_simt: bool = False, slopes: Optional[torch.Tensor] = None,
                     items: Optional[torch.Tensor] = None) -> None:
    """Attention of sequences with one query token each: the tensor-core kernel (csrc/attention_decode_mma.cu)
    where it takes the shape, else the CUDA-core kernel's split form (always, when score biases are given).  Same
    partial-workspace layout.  ``items``: the step's list of live (sequence, kv head, split) items from
    :func:`attention_decode_items`, which a caller with several layers builds once per step; built here if not given."""
    if force_simt or slopes is not None or not attention_decode_fast_ok(q.dtype, n_q, n_kv, head_dim, page_size):
        attention_simt(q, out, cache, block_table, q_start, kv_len, work, n_work, n_q, n_kv, head_dim, page_size, window,
                       scale, True, status, split_keys=split_keys, max_splits=max_splits, split_start=split_start,
                       total_splits=total_splits, partial=partial, slopes=slopes)
        return
    _cuda(q, out, cache, block_table, q_start, kv_len, work, status, partial, split_start)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or not cache.is_contiguous():
        raise KernelError("attention_decode: q, out and cache must be bfloat16 and the cache contiguous")
    if tuple(cache.shape[1:]) != (2, n_kv, page_size, head_dim):
        raise KernelError(f"attention_decode: cache shape {tuple(cache.shape)} is not [pages, 2, {n_kv}, {page_size}, {head_dim}]")
    for name, t in (("block_table", block_table), ("q_start", q_start), ("kv_len", kv_len), ("work", work),
                    ("split_start", split_start)):
        if t.dtype != torch.int32:
            raise KernelError(f"attention_decode: {name} must be int32")
    slots = _partial_slots(partial, total_splits, n_q, head_dim, "attention_decode")
    if items is None:
        items = torch.empty(n_work * n_kv * max_splits, dtype=torch.int32, device=q.device)
        attention_decode_items(split_start, n_work, n_kv, max_splits, items)
    elif items.dtype != torch.int32 or not items.is_cuda or not items.is_contiguous():
        raise KernelError("attention_decode: items must be a contiguous int32 device tensor")
    _check(bf16lib().rs_attention_decode_bf16(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cache), cache.stride(0), cache.shape[0], page_size,
        _ptr(block_table), block_table.stride(0), _ptr(q_start), _ptr(kv_len), _ptr(work), n_work, n_q, n_kv, head_dim,
        int(window), float(scale), split_keys, max_splits, _ptr(split_start), _ptr(items), _ptr(partial), slots, _ptr(status),
        _stream()), "attention_decode_bf16", 2)


def attention_decode_items(split_start: torch.Tensor, n_work: int, n_kv: int, max_splits: int, items: torch.Tensor) -> None:
    """items[id] for every live (sequence, kv head, split) of a step of single tokens, id as the tensor-core decode
    kernel counts them; ``items`` int32 with room for split_start[n_work] * n_kv entries (n_work * n_kv * max_splits
    always suffices).  One small kernel; its result serves every layer of the step."""
    _cuda(split_start, items)
    if split_start.dtype != torch.int32 or items.dtype != torch.int32 or not items.is_contiguous() or split_start.numel() < n_work + 1:
        raise KernelError("attention_decode_items: int32 tensors, split_start with n_work + 1 entries")
    _check(bf16lib().rs_attention_decode_build_items(_ptr(split_start), n_work, n_kv, max_splits, _ptr(items), _stream()),
           "attention_decode_items")


# ----------------------------------------------------------------------------- the bounded-wait probe
def wait_probe(status: torch.Tensor) -> dict:
    """Runs the probe kernel of csrc/wait_probe.cu (a wait nobody satisfies, limit 2 ms) with ``status`` as its status
    word and returns {"satisfied": bool, "waited_us": int, "limit_us": int} once it has ended.  For tests."""
    lib = load_library("probe")
    lib.rs_wait_probe.argtypes = [c_void_p, c_void_p, c_void_p]
    lib.rs_wait_probe_limit_ns.restype = ctypes.c_ulonglong
    _cuda(status)
    outcome = torch.full((2,), -1, dtype=torch.int32, device=status.device)
    _check(lib.rs_wait_probe(_ptr(status), _ptr(outcome), _stream()), "wait_probe")
    got = outcome.cpu().tolist()
    return {"satisfied": got[0] == 1, "waited_us": got[1], "limit_us": int(lib.rs_wait_probe_limit_ns() // 1000)}


# ----------------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, n_rows: int, out: torch.Tensor, status: torch.Tensor,
           temps: Optional[torch.Tensor] = None, uniforms: Optional[torch.Tensor] = None) -> None:
    """out[r] = argmax of row r when temps is None or temps[r] <= 0, else a draw at temperature temps[r]."""
    _cuda(logits, out, status, temps, uniforms)
    _rows_contiguous(logits, "logits")
    if logits.dtype != torch.float32 or out.dtype != torch.int32 or out.numel() < n_rows:
        raise KernelError("sample: logits float32, out int32 with n_rows entries")
    if temps is not None and (uniforms is None or temps.dtype != torch.float32 or uniforms.dtype != torch.float32):
        raise KernelError("sample: temps and uniforms must both be float32")
    _check(core().rs_sample(_ptr(logits), logits.stride(0), n_rows, logits.shape[1], _ptr(temps), _ptr(uniforms),
                            _ptr(out), _ptr(status), _stream()), "sample")
