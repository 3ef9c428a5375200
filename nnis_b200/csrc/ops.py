"""Python face of the CUDA entry points.

Each function checks dtypes, shapes, contiguity and device before it hands raw
pointers to the library, and turns a non-zero return code into an exception: a
size that a kernel does not take is refused with a message, never run.  Nothing
here computes; without the compiled library nothing works, on purpose.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build as _build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}
_ARG_ERRORS = {-1: "bad argument", -2: "unsupported size or dtype", -3: "misaligned pointer",
               -4: "a kernel reported an error status"}


class KernelError(RuntimeError):
    pass


_launches = 0


def launch_count() -> int:
    """Kernels of this library launched (or captured) so far in this process."""
    return _launches


def _lib() -> ctypes.CDLL:
    return _build.load()


def _check(code: int, what: str, kernels: int = 1) -> None:
    global _launches
    if code == 0:
        _launches += kernels
        return
    if code < 0:
        raise KernelError(f"{what}: {_ARG_ERRORS.get(code, 'error')} (code {code})")
    raise KernelError(f"{what}: CUDA error {code} at launch")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> ctypes.c_void_p:
    """The current stream's handle (the raw getter is some ten microseconds
    cheaper than building a Stream object, and a decode step asks several times)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None:
            _need(t.is_cuda, "kernels take CUDA tensors only (there is no CPU path)")
            _need(t.is_contiguous(), "kernels take contiguous tensors")


def code_of(dtype: torch.dtype) -> int:
    _need(dtype in _DTYPE_CODE, f"dtype {dtype} is not supported (float32 or bfloat16)")
    return _DTYPE_CODE[dtype]


# ---------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, hidden: torch.Tensor,
          status: torch.Tensor) -> None:
    """hidden[n] = table[tokens[n]] widened to float32; an id outside the table
    sets ``status[0]`` and yields a zero row."""
    _cuda(table, tokens, hidden, status)
    n, width = hidden.shape
    _need(tokens.dtype == torch.int32 and tokens.numel() >= n, "tokens: int32 [n]")
    _need(hidden.dtype == torch.float32 and table.shape[1] == width, "hidden: float32 [n, width]")
    _need(status.dtype == torch.int32, "status: int32")
    _check(_lib().nnis_embed(_ptr(table), code_of(table.dtype), _ptr(tokens), _ptr(hidden), n, width,
                             table.shape[0], _ptr(status), _stream()), "embed")


def copy_async(dst: torch.Tensor, src: torch.Tensor) -> None:
    """dst <- src on the current stream, both contiguous and equally large; the host
    side of the pair must be pinned memory for the copy to be asynchronous."""
    _need(dst.is_contiguous() and src.is_contiguous(), "copy_async: contiguous tensors")
    nbytes = src.numel() * src.element_size()
    _need(nbytes == dst.numel() * dst.element_size(), "copy_async: sizes differ")
    code = _lib().nnis_copy_async(_ptr(dst), _ptr(src), ctypes.c_longlong(nbytes), _stream())
    if code != 0:
        raise KernelError(f"copy_async: CUDA error {code}")


def stream_synchronize() -> None:
    """Wait for the current stream (what ``Stream.synchronize`` does, without the object)."""
    code = _lib().nnis_stream_synchronize(_stream())
    if code != 0:
        raise KernelError(f"stream_synchronize: CUDA error {code}")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * weight, statistics in float32."""
    _cuda(x, weight, out, rows)
    n, width = out.shape
    _need(x.dtype == torch.float32 and x.shape[1] == width, "x: float32 [*, width]")
    _need(weight.dtype == torch.float32 and weight.numel() == width, "weight: float32 [width]")
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.numel() >= n, "rows: int32 [n]")
    else:
        _need(x.shape[0] >= n, "x has fewer rows than out")
    _check(_lib().nnis_rmsnorm(_ptr(x), _ptr(rows), _ptr(weight), _ptr(out), code_of(out.dtype), n,
                               width, ctypes.c_float(eps), PDL, _stream()), "rmsnorm")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:], gate_up float32 [n, 2I]."""
    _cuda(gate_up, out)
    n, inter = out.shape
    _need(gate_up.dtype == torch.float32 and tuple(gate_up.shape) == (n, 2 * inter),
          "gate_up: float32 [n, 2 * inter]")
    _check(_lib().nnis_silu_mul(_ptr(gate_up), _ptr(out), code_of(out.dtype),
                                ctypes.c_longlong(n), inter, _stream()), "silu_mul")


def rope_store(qkv: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor,
               page_table: Optional[torch.Tensor], cos: Optional[torch.Tensor],
               sin: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
               v_cache: Optional[torch.Tensor], heads: int, kv_heads: int, head_dim: int,
               page_size: int) -> None:
    """Rotate q and k heads of packed rows in place, store k and v in the cache.
    ``kv_heads == 0``: the rows hold q only and nothing is stored."""
    _cuda(qkv, token_pos, token_seq, page_table, cos, sin, k_cache, v_cache)
    n = qkv.shape[0]
    _need(qkv.shape[1] == (heads + 2 * kv_heads) * head_dim, "qkv: [n, (heads + 2 kv_heads) * d]")
    _need(token_pos.dtype == torch.int32 and token_seq.dtype == torch.int32, "positions: int32")
    cols = 0
    if kv_heads > 0:
        _need(page_table is not None and page_table.dtype == torch.int32, "page_table: int32")
        _need(k_cache is not None and k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype,
              "cache dtype differs from qkv")
        _need(tuple(k_cache.shape[1:]) == (kv_heads, page_size, head_dim), "cache: [pages, kv, page, d]")
        cols = page_table.shape[1]
    rotate = 0
    if cos is not None:
        _need(cos.dtype == torch.float32 and cos.shape[1] == head_dim // 2, "cos/sin: float32 [C, d/2]")
        rotate = 1
    _check(_lib().nnis_rope_store(_ptr(qkv), code_of(qkv.dtype), _ptr(token_pos), _ptr(token_seq),
                                  _ptr(page_table), cols, _ptr(cos), _ptr(sin), _ptr(k_cache),
                                  _ptr(v_cache), n, heads, kv_heads, head_dim, page_size, rotate,
                                  _stream()), "rope_store")


STORE, STORE_F32, ADD_F32 = 0, 1, 2


def gemm_simt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
              mode: int) -> None:
    """out (op)= a . w^T + bias on the CUDA cores; float32 accumulation."""
    _cuda(a, w, bias, out)
    m, k = a.shape
    n = w.shape[0]
    _need(w.shape[1] == k and a.dtype == w.dtype, "gemm: a [m, k], w [n, k] of one dtype")
    _need(tuple(out.shape) == (m, n), "gemm: out [m, n]")
    _need(out.dtype == (a.dtype if mode == STORE else torch.float32), "gemm: out dtype vs mode")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n, "gemm: bias float32 [n]")
    _check(_lib().nnis_gemm_simt(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), m, n, k, code_of(a.dtype),
                                 mode, _stream()), "gemm_simt")


def attention_generic(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      token_pos: torch.Tensor, token_seq: torch.Tensor, page_table: torch.Tensor,
                      out: torch.Tensor, heads: int, kv_heads: int, head_dim: int, window: int,
                      scale: float, n_splits: int = 1,
                      partial: Optional[torch.Tensor] = None) -> None:
    """Causal attention of packed query tokens over the paged cache."""
    _cuda(k_cache, v_cache, token_pos, token_seq, page_table, out, partial)
    _need(q.is_cuda, "q: CUDA tensor")
    n = out.shape[0]
    pages, nkv, page_size, d = k_cache.shape
    _need(nkv == kv_heads and d == head_dim, "cache shape differs from the heads given")
    _need(head_dim % 2 == 0 and 2 <= head_dim <= 256,
          f"attention: head_dim {head_dim} is not an even size in 2..256")
    _need(heads % kv_heads == 0, "attention: heads is not a multiple of kv_heads")
    _need(pages * nkv * page_size < 2 ** 31, "attention: the cache has too many rows")
    _need(out.shape[1] == heads * head_dim and out.dtype == k_cache.dtype == q.dtype,
          "attention: out [n, heads * d] in the cache dtype")
    if n_splits > 1:
        _need(partial is not None and partial.dtype == torch.float32
              and partial.numel() >= n * heads * n_splits * (head_dim + 2),
              "attention: partial scratch too small")
    _check(_lib().nnis_attention_generic(
        _ptr(q), q_stride, _ptr(k_cache), _ptr(v_cache), _ptr(token_pos), _ptr(token_seq),
        _ptr(page_table), page_table.shape[1], _ptr(out), _ptr(partial), n, heads, kv_heads, head_dim,
        page_size, window, ctypes.c_float(scale), n_splits, code_of(out.dtype), _stream()),
        "attention_generic", 2 if n_splits > 1 else 1)


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(logits, out)
    _need(logits.dtype == torch.float32 and out.dtype == torch.int32, "argmax: float32 -> int32")
    n, vocab = logits.shape
    _need(out.numel() >= n, "argmax: out too small")
    _check(_lib().nnis_argmax(_ptr(logits), _ptr(out), n, vocab, _stream()), "argmax")


def sample_temperature(logits: torch.Tensor, temperature: torch.Tensor, rng_state: torch.Tensor,
                       out: torch.Tensor) -> None:
    """One seeded draw per row; ``rng_state`` (int64, SplitMix64) advances."""
    _cuda(logits, temperature, rng_state, out)
    n, vocab = logits.shape
    _need(logits.dtype == torch.float32 and out.dtype == torch.int32, "sample: float32 -> int32")
    _need(temperature.dtype == torch.float32 and temperature.numel() >= n, "temperature: float32 [n]")
    _need(rng_state.dtype == torch.int64 and rng_state.numel() >= n, "rng_state: int64 [n]")
    _check(_lib().nnis_sample_temperature(_ptr(logits), _ptr(temperature), _ptr(rng_state),
                                          _ptr(out), n, vocab, _stream()), "sample_temperature")


EPI_STORE, EPI_STORE_F32, EPI_ADD_F32, EPI_GATED, EPI_QKV, EPI_ARGMAX = 0, 1, 2, 3, 4, 5
# activations that the storing epilogues of the bfloat16 products can apply (gelu with erf, its tanh form)
GEMM_ACT_RELU2, GEMM_ACT_GELU_ERF, GEMM_ACT_GELU_TANH = 1, 2, 3
# programmatic dependent launch between the decode kernels (NNIS_PDL=0 turns it off)
PDL = 0 if os.environ.get("NNIS_PDL", "1") == "0" else 1
# The QKV projection of a decode step lets attention_decode_tma start with it instead of after
# its own wait, so that the copies of old pages run under it (NNIS_EARLY_RELEASE=0: off)
EARLY_RELEASE = 0 if os.environ.get("NNIS_EARLY_RELEASE", "1") == "0" else 1
_status = {}


def status_word(device) -> torch.Tensor:
    """One int32 per device that kernels set when a bounded wait runs out."""
    key = torch.device(device).index or 0
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def check_status(device) -> None:
    """Raise if a kernel gave up a wait since the last check (synchronises)."""
    word = status_word(device)
    if int(word.item()) != 0:
        word.zero_()
        raise KernelError("a kernel gave up waiting for an asynchronous copy; results are invalid")


def gemv_grid(m: int, n: int, k: int, device) -> int:
    return int(_lib().nnis_gemv_grid(m, n, k, sm_count(device)))
_sm_count = {}


def sm_count(device) -> int:
    key = torch.device(device).index or 0
    if key not in _sm_count:
        _sm_count[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_count[key]


# The decode projections have two kernels: one whose CTAs hold all rows of x for eight
# output features each (at most 64 rows), and one that cuts the rows into tiles of 16
# (more than 16 rows, few output features, every CTA resident at once).  Where only the
# first applies, the parts choose it up to DECODE_GEMV_ROWS rows, and fold the norm before
# a projection into it up to GEMV_NORM_ROWS rows: every CTA of that kernel normalises all
# rows for itself, through registers, which with more than a tile of rows costs more than
# a norm kernel of its own.  Beyond that the general kernels (tcgen05) run.
DECODE_GEMV_ROWS = int(os.environ.get("NNIS_DECODE_GEMV_ROWS", "48"))
GEMV_NORM_ROWS = int(os.environ.get("NNIS_GEMV_NORM_ROWS", "16"))
# Most wanted rows for which the head runs as the decode projection kernel (with the final
# norm and the greedy pick folded in); with more, its products on mma.sync tiles cost more
# than the weights' way from memory, and the norm, the tcgen05 product and the pick run
# as kernels of their own.
GEMV_HEAD_ROWS = int(os.environ.get("NNIS_GEMV_HEAD_ROWS", "48"))


def gemv_kind(m: int, n: int, k: int, epilogue: int = EPI_STORE, device=None, normed: bool = False,
              rows_kernel: bool = True, shared_norm: bool = False) -> int:
    """Which decode projection kernel runs this product: 2 the one over tiles of rows, 1
    the one whose CTAs hold all rows, 0 neither (the general kernels must run).
    ``rows_kernel=False``: as if the first did not exist.  ``shared_norm``: with the norm
    before it begun by the projection before that (see ``gemv_bf16``'s ``emit``)."""
    sms = sm_count(device) if device is not None else 148
    if shared_norm:
        return int(_lib().nnis_gemv_kind(m, n, k, epilogue, 2, sms)) if rows_kernel else 0
    if not rows_kernel:
        return int(_lib().nnis_gemv_units_takes(m, n, k, epilogue, 1 if normed else 0, sms))
    return int(_lib().nnis_gemv_kind(m, n, k, epilogue, 1 if normed else 0, sms))


# A norm between two decode projections, shared out between them (both halves or neither).
# (bit 0: the norm before a gated feed-forward, bit 1: the norm before q, k, v)
SHARED_NORM = int(os.environ.get("NNIS_SHARED_NORM", "3"))


def gemv_shares_norm(m: int, n: int, k: int, epilogue: int, device=None) -> bool:
    """Whether the decode projection of these sizes can take its input from the epilogue of
    the projection before it (``gemv_bf16`` with ``emit`` there and ``shares`` here)."""
    return bool(SHARED_NORM & (2 if epilogue == EPI_QKV else 1)) \
        and gemv_kind(m, n, k, epilogue, device, shared_norm=True) == 2


def gemv_takes(m: int, n: int, k: int, epilogue: int = EPI_STORE, device=None, normed: bool = False) -> bool:
    """Whether a decode projection kernel can run this shape: K in steps of 16, N in
    steps of 8, operands that fit shared memory; at most 64 rows, or up to 128 where the
    kernel over tiles of rows applies."""
    return gemv_kind(m, n, k, epilogue, device, normed) > 0


def gemv_pays(m: int, n: int, k: int, epilogue: int = EPI_STORE, device=None, normed: bool = False) -> bool:
    """Whether the parts of a decode step should choose a decode projection kernel for
    this product (see the thresholds above)."""
    kind = gemv_kind(m, n, k, epilogue, device, normed)
    return kind == 2 or (kind == 1 and m <= DECODE_GEMV_ROWS and (not normed or m <= GEMV_NORM_ROWS))


def gemv_slices(m: int, n: int, k: int, device=None, rows_kernel: bool = True) -> int:
    """Launches that an ADD_F32 product of these sizes takes (slices of K, each
    adding its share in order); 0: not taken."""
    sms = sm_count(device) if device is not None else 148
    if not rows_kernel:
        return int(_lib().nnis_gemv_units_slices(m, n, k, sms))
    return int(_lib().nnis_gemv_slices(m, n, k, sms))


def gemv_bf16(w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, epilogue: int,
              x: Optional[torch.Tensor] = None, hidden: Optional[torch.Tensor] = None,
              norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0,
              rows: Optional[torch.Tensor] = None, m: Optional[int] = None,
              token_pos: Optional[torch.Tensor] = None, token_seq: Optional[torch.Tensor] = None,
              page_table: Optional[torch.Tensor] = None, cos: Optional[torch.Tensor] = None,
              sin: Optional[torch.Tensor] = None, k_cache: Optional[torch.Tensor] = None,
              v_cache: Optional[torch.Tensor] = None, heads: int = 0, kv_heads: int = 0,
              head_dim: int = 0, page_size: int = 0, logits: Optional[torch.Tensor] = None,
              scratch: Optional[torch.Tensor] = None, next_tokens: Optional[torch.Tensor] = None,
              next_pos: Optional[torch.Tensor] = None, release_early: bool = False,
              rows_kernel: bool = True, emit: Optional[tuple] = None,
              shares: Optional[torch.Tensor] = None, act: int = 0) -> None:
    """A decode-step projection with its prologue and epilogue fused (at most 64
    rows).  The input is ``x`` (bfloat16 [m, k]) or ``hidden`` (float32 residual
    rows, normed with ``norm_weight``/``eps`` on the way in; ``rows`` picks them).
    EPI_ARGMAX writes
    int32 picks to ``out``; ``scratch`` (int32, ``argmax_scratch_ints``) is its
    workspace, ``logits`` optional, ``next_tokens``/``next_pos`` the decode state.
    ``release_early``: the kernel launched after this one may start together with it
    (only for a successor that reads, before its own wait, nothing that a kernel of
    the step writes: attention_decode_tma).  ``rows_kernel=False``: the kernel whose CTAs
    hold all rows even where the one over tiles of rows applies (for comparisons).

    A norm between two projections can be shared out between them.  ``emit`` (EPI_ADD_F32)
    is ``(x_next, norm_weight, shares)``: the epilogue also writes the rows it has summed,
    times ``norm_weight`` (float32 [n]), to ``x_next`` (bfloat16 [m, n]) and every eight
    columns' sum of squares to ``shares`` (float32 [m, n / 8]).  The projection after it
    takes ``x=x_next, shares=shares, eps=`` the norm's, and scales its sums by
    ``1 / sqrt(mean of squares + eps)`` (``gemv_shares_norm`` says whether it can)."""
    _cuda(w, bias, out, x, hidden, norm_weight, rows, token_pos, token_seq, page_table, cos, sin,
          k_cache, v_cache, logits, scratch, next_tokens, next_pos, shares, *(emit or ()))
    n, k = w.shape
    _need(w.dtype == torch.bfloat16, "gemv: bfloat16 weights")
    if hidden is not None:
        _need(hidden.dtype == torch.float32 and hidden.shape[1] == k, "gemv: hidden float32 [*, k]")
        _need(norm_weight is not None and norm_weight.dtype == torch.float32
              and norm_weight.numel() == k, "gemv: norm weight float32 [k]")
        rows_m = rows.numel() if rows is not None else hidden.shape[0]
        m = rows_m if m is None else m
        if rows is not None:
            _need(rows.dtype == torch.int32, "gemv: rows int32")
    else:
        _need(x is not None and x.dtype == torch.bfloat16 and x.shape[1] == k, "gemv: x bfloat16 [m, k]")
        m = x.shape[0] if m is None else m
    if shares is not None:
        _need(hidden is None and eps > 0.0, "gemv: shares come with x and the norm's eps")
        _need(shares.dtype == torch.float32 and tuple(shares.shape) == (m, k // 8) and shares.is_contiguous(),
              "gemv: shares float32 [m, k / 8]")
        _need(gemv_kind(m, n, k, epilogue, w.device, rows_kernel=rows_kernel, shared_norm=True) == 2,
              f"gemv: shape m={m} n={n} k={k} takes no shared norm")
    else:
        _need(gemv_kind(m, n, k, epilogue, w.device, hidden is not None, rows_kernel) > 0,
              f"gemv: shape m={m} n={n} k={k} is not taken")
    emit_x = emit_w = emit_ss = None
    if emit is not None:
        emit_x, emit_w, emit_ss = emit
        _need(epilogue == EPI_ADD_F32, "gemv: only the adding epilogue emits")
        _need(emit_x.dtype == torch.bfloat16 and tuple(emit_x.shape) == (m, n) and emit_x.is_contiguous(),
              "gemv: emit x bfloat16 [m, n]")
        _need(emit_w.dtype == torch.float32 and emit_w.numel() == n, "gemv: emit weight float32 [n]")
        _need(emit_ss.dtype == torch.float32 and tuple(emit_ss.shape) == (m, n // 8) and emit_ss.is_contiguous(),
              "gemv: emit shares float32 [m, n / 8]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n, "gemv: bias float32 [n]")
    _need(act == 0 or (epilogue == EPI_STORE and act in (GEMM_ACT_RELU2, GEMM_ACT_GELU_ERF, GEMM_ACT_GELU_TANH)),
          "gemv: an activation goes with the storing epilogue")
    if epilogue == EPI_STORE:
        _need(out.dtype == torch.bfloat16 and tuple(out.shape) == (m, n), "gemv: out bfloat16 [m, n]")
    elif epilogue in (EPI_STORE_F32, EPI_ADD_F32):
        _need(out.dtype == torch.float32 and tuple(out.shape) == (m, n), "gemv: out float32 [m, n]")
    elif epilogue == EPI_GATED:
        _need(out.dtype == torch.bfloat16 and tuple(out.shape) == (m, n // 2),
              "gemv: out bfloat16 [m, n / 2]")
    elif epilogue == EPI_QKV:
        _need(n == (heads + 2 * kv_heads) * head_dim and head_dim % 16 == 0, "gemv: qkv rows")
        _need(out.dtype == torch.bfloat16 and tuple(out.shape) == (m, heads * head_dim),
              "gemv: q out bfloat16 [m, heads * d]")
        _need(token_pos is not None and token_pos.dtype == torch.int32 and token_pos.numel() >= m,
              "gemv: token_pos int32 [m]")
        if kv_heads > 0:
            _need(k_cache is not None and k_cache.dtype == torch.bfloat16
                  and tuple(k_cache.shape[1:]) == (kv_heads, page_size, head_dim)
                  and page_table is not None and token_seq is not None, "gemv: cache [pages, kv, page, d]")
        if cos is not None:
            _need(cos.dtype == torch.float32 and cos.shape[1] == head_dim // 2, "gemv: cos/sin tables")
    elif epilogue == EPI_ARGMAX:
        _need(out.dtype == torch.int32 and out.numel() >= m, "gemv: picks int32 [m]")
        _need(scratch is not None and scratch.dtype == torch.int32
              and scratch.numel() >= argmax_scratch_ints(m, n, k, w.device), "gemv: argmax scratch")
        if logits is not None:
            _need(logits.dtype == torch.float32 and tuple(logits.shape) == (m, n), "gemv: logits [m, n]")
        if next_tokens is not None:
            _need(next_pos is not None and next_tokens.dtype == next_pos.dtype == torch.int32
                  and next_tokens.numel() >= m and next_pos.numel() >= m, "gemv: decode state int32")
    else:
        raise KernelError(f"gemv: unknown epilogue {epilogue}")
    cols = page_table.shape[1] if page_table is not None else 0
    best_val = best_idx = ticket = 0
    if epilogue == EPI_ARGMAX:
        grid = gemv_grid(m, n, k, w.device)
        base = scratch.data_ptr()
        ticket, best_val, best_idx = base, base + 16, base + 16 + 4 * m * grid
    _check(_lib().nnis_gemv_bf16(
        _ptr(x), _ptr(hidden), _ptr(rows), _ptr(norm_weight), ctypes.c_float(eps), _ptr(w), _ptr(bias), _ptr(out), m, n, k, epilogue, _ptr(token_pos), _ptr(token_seq),
        _ptr(page_table), cols, _ptr(cos), _ptr(sin), _ptr(k_cache), _ptr(v_cache), heads, kv_heads,
        head_dim, page_size, _ptr(logits), ctypes.c_void_p(best_val), ctypes.c_void_p(best_idx),
        ctypes.c_void_p(ticket), _ptr(next_tokens), _ptr(next_pos), _ptr(emit_x), _ptr(emit_w),
        _ptr(emit_ss), _ptr(shares), act, _ptr(status_word(w.device)),
        sm_count(w.device),
        PDL | (2 if release_early and PDL and EARLY_RELEASE else 0) | (0 if rows_kernel else 4), _stream()),
        "gemv_bf16",
        gemv_slices(m, n, k, w.device, rows_kernel) if epilogue == EPI_ADD_F32 and hidden is None else 1)


def argmax_scratch_ints(m: int, n: int, k: int, device) -> int:
    """int32 words of scratch for EPI_ARGMAX: a ticket, then per-CTA bests.  The
    buffer must be zero before its first use (the kernel re-zeroes the ticket)."""
    return 4 + 2 * m * gemv_grid(m, n, k, device)


def attention_decode(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     token_pos: torch.Tensor, token_seq: torch.Tensor, page_table: torch.Tensor,
                     out: torch.Tensor, heads: int, kv_heads: int, head_dim: int, window: int,
                     scale: float, n_splits: int = 1, partial: Optional[torch.Tensor] = None,
                     merge: bool = True) -> None:
    """One query token per sequence over the paged bfloat16 cache.  With
    ``merge=False`` and several splits, ``partial`` is left for the consumer."""
    _cuda(k_cache, v_cache, token_pos, token_seq, page_table, out, partial)
    _need(q.is_cuda and q.dtype == torch.bfloat16 == k_cache.dtype == out.dtype,
          "attention_decode: bfloat16 tensors")
    n = out.shape[0]
    pages, nkv, page_size, d = k_cache.shape
    _need(nkv == kv_heads and d == head_dim, "cache shape differs from the heads given")
    _need(head_dim % 16 == 0 and 16 <= head_dim <= 256,
          f"attention: head_dim {head_dim} is not a multiple of 16 in 16..256")
    _need(heads % kv_heads == 0, "attention: heads is not a multiple of kv_heads")
    _need(pages * nkv * page_size < 2 ** 31, "attention: the cache has too many rows")
    _need(out.shape[1] == heads * head_dim and n <= 65535, "attention_decode: out [n <= 65535, heads * d]")
    if n_splits > 1:
        _need(partial is not None and partial.dtype == torch.float32
              and partial.numel() >= n * heads * n_splits * (head_dim + 2),
              "attention: partial scratch too small")
    _check(_lib().nnis_attention_decode(
        _ptr(q), q_stride, _ptr(k_cache), _ptr(v_cache), _ptr(token_pos), _ptr(token_seq),
        _ptr(page_table), page_table.shape[1], _ptr(out), _ptr(partial), n, heads, kv_heads, head_dim,
        page_size, window, ctypes.c_float(scale), n_splits, 1 if merge else 0,
        _ptr(status_word(out.device)), PDL, _stream()),
        "attention_decode", 2 if n_splits > 1 and merge else 1)


def attention_decode_takes(head_dim: int) -> bool:
    """Head sizes of the CUDA-core decode kernel (whole 32-byte pieces of a row per lane)."""
    return head_dim % 16 == 0 and 16 <= head_dim <= 256


# Whether the decode attention kernel for few sequences asks the same pages of the layer that
# runs next into L2 when it is through with its own (batch 8 of the 135M shape: +2 %).
KV_PREFETCH = os.environ.get("NNIS_KV_PREFETCH", "1") == "1"
PREFILL_SHORT_CHUNKS = os.environ.get("NNIS_PREFILL_SHORT_CHUNKS", "1") == "1"
TMA_SLICE_PAGES = int(os.environ.get("NNIS_TMA_SLICE_PAGES", "0"))  # 0: chosen by the plan
TMA_ATTENTION = 0 if os.environ.get("NNIS_TMA_ATTENTION", "1") == "0" else 1
_tma_ctas_per_sm: dict = {}


def attention_decode_tma_max_pages(head_dim: int) -> int:
    """Pages of one slice that attention_decode_tma holds (all at once, in shared memory)."""
    return int(_lib().nnis_attention_decode_tma_max_pages(int(head_dim)))


def tma_slices(groups: int, table_cols: int, sms: int, most_pages: int, fit, fixed_pages: int = 0) -> int:
    """The rule behind ``attention_decode_tma_plan``, free of the device: ``groups`` CTAs per
    slice (sequences x kv heads x tiles of query heads), ``table_cols`` pages to cut, ``sms``
    SMs, at most ``most_pages`` pages a slice, and ``fit(pages)`` the CTAs of that many pages
    that one SM holds at once.  Returns the number of slices, 0: not for this kernel."""
    def plan(pages: int):
        splits = min(128, -(-table_cols // pages))
        per = -(-table_cols // splits)
        if per > most_pages:
            return 0, 0, 0
        return splits, groups * splits, fit(per)

    if fixed_pages:
        splits, ctas, room = plan(fixed_pages)
        return splits if 0 < ctas <= room * sms else 0
    splits, ctas, room = plan(4)
    if splits > 16:
        # The slice that arrives last asks for 16 partial records a trip to L2: beyond 16 slices
        # (contexts beyond 4,096) the longest slices whose CTAs are still all resident, eight pages
        # one to an SM or six pages two to an SM (one sequence at context 16,384: 0.592 -> 0.512 ms
        # a step, two at 8,192: 0.540 -> 0.493)
        for pages in (8, 6):
            long_splits, long_ctas, long_room = plan(pages)
            if 0 < long_ctas <= min(long_room, 2) * sms:
                return long_splits
    if ctas > 2 * sms:
        wide, wide_ctas, wide_room = plan(6)
        if 0 < wide_ctas <= min(wide_room, 2) * sms:
            return wide
    return splits if 0 < ctas <= room * sms else 0


def attention_decode_tma_plan(n: int, heads: int, kv_heads: int, head_dim: int, page_size: int,
                              table_cols: int, device, share: int = 1) -> int:
    """Into how many slices attention_decode_tma cuts ``table_cols`` pages for a step of ``n``
    sequences, or 0 when the step is not for that kernel: it takes head sizes 64 and 128 and
    only steps whose CTAs are all resident together (few sequences, or short contexts);
    other steps stream their slices through the ring of attention_decode_mma.  Slices are of
    four pages (more for page tables beyond 128 x 4 columns, up to what fits; with more than 16
    slices of four pages, of eight or six pages where those CTAs are resident); when four pages make
    more CTAs than two per SM, of six pages if those CTAs are resident two to an SM: fewer
    partial records and fewer CTAs that wait for room beside the projection's (batch 8 of the
    135M shape: 0.637 -> 0.618 ms a step; at batch 1, where CTAs are few, four pages are
    4 % ahead).  ``share``: steps that run side by side on the device.
    ``NNIS_TMA_SLICE_PAGES`` fixes the pages of a slice."""
    if not TMA_ATTENTION or head_dim not in (64, 128) or page_size != 64 or n > 65535:
        return 0
    groups = n * kv_heads * (-(-(heads // kv_heads) // 16))
    sms = sm_count(device) // max(1, share)

    def fit(pages: int) -> int:
        key = (head_dim, pages, torch.device(device).index or 0)
        if key not in _tma_ctas_per_sm:
            _tma_ctas_per_sm[key] = int(_lib().nnis_attention_decode_tma_ctas_per_sm(head_dim, pages))
        return _tma_ctas_per_sm[key]

    return tma_slices(groups, table_cols, sms, attention_decode_tma_max_pages(head_dim), fit, TMA_SLICE_PAGES)


def attention_decode_tma(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         token_pos: torch.Tensor, token_seq: torch.Tensor, page_table: torch.Tensor,
                         out: torch.Tensor, heads: int, kv_heads: int, head_dim: int, window: int,
                         scale: float, n_splits: int, partial: Optional[torch.Tensor] = None,
                         tickets: Optional[torch.Tensor] = None, ahead: int = 0) -> None:
    """Decode attention with every page of a slice in shared memory at once (``n_splits``
    from ``attention_decode_tma_plan``): pages by TMA, a warp per page.  Scratch as for
    ``attention_decode_mma``.  ``ahead``: elements from these caches to the ones read next
    (the next layer's), whose same pages the kernel asks into L2; 0: none."""
    _cuda(k_cache, v_cache, token_pos, token_seq, page_table, out, partial, tickets)
    _need(q.is_cuda and q.dtype == torch.bfloat16 == k_cache.dtype == out.dtype,
          "attention_decode_tma: bfloat16 tensors")
    n = out.shape[0]
    pages, nkv, page_size, d = k_cache.shape
    _need(nkv == kv_heads and d == head_dim, "cache shape differs from the heads given")
    _need(head_dim in (64, 128) and page_size == 64, "attention_decode_tma: head size 64 or 128, pages of 64")
    _need(heads % kv_heads == 0, "attention: heads is not a multiple of kv_heads")
    _need(pages * nkv * page_size < 2 ** 31, "attention: the cache has too many rows")
    _need(out.shape[1] == heads * head_dim and n <= 65535, "attention: out [n <= 65535, heads * d]")
    most = attention_decode_tma_max_pages(head_dim)
    _need(1 <= n_splits <= 128 and -(-page_table.shape[1] // n_splits) <= most,
          f"attention_decode_tma: at most 128 slices of at most {most} pages")
    if n_splits > 1:
        _need(partial is not None and partial.dtype == torch.float32
              and partial.numel() >= n * heads * n_splits * (head_dim + 2),
              "attention: partial scratch too small")
        _need(tickets is not None and tickets.dtype == torch.int32
              and tickets.numel() >= mma_ticket_count(n, heads, kv_heads), "attention: tickets")
    _check(_lib().nnis_attention_decode_tma(
        _ptr(q), q_stride, _ptr(k_cache), _ptr(v_cache), ctypes.c_longlong(pages * nkv * page_size),
        _ptr(token_pos), _ptr(token_seq), _ptr(page_table), page_table.shape[1], _ptr(out),
        _ptr(partial), _ptr(tickets), n, heads, kv_heads, head_dim, page_size, window,
        ctypes.c_float(scale), n_splits, ctypes.c_longlong(ahead), _ptr(status_word(out.device)), PDL,
        _stream()),
        "attention_decode_tma")


def attention_decode_mma_takes(head_dim: int, page_size: int) -> bool:
    return head_dim in (64, 128) and page_size == 64


_decode_mma_resident: dict = {}
# 1: the decode attention may run with one stage less where the wave model favours it
DECODE_STAGE_CHOICE = int(os.environ.get("NNIS_DECODE_STAGE_CHOICE", "1")) \
    and os.environ.get("NNIS_DECODE_FILL") is None


def attention_decode_mma_stages(head_dim: int) -> int:
    """Pages of K and V that a CTA of the tensor-core decode kernel keeps in flight by default."""
    return int(_lib().nnis_attention_decode_mma_stages(int(head_dim)))


def attention_decode_mma_resident(head_dim: int, device, stages: int = 0) -> int:
    """How many CTAs of the tensor-core decode kernel the device holds at once
    (``stages`` pages in flight per CTA; 0: the default)."""
    key = (head_dim, torch.device(device).index or 0, stages)
    if key not in _decode_mma_resident:
        per_sm = int(_lib().nnis_attention_decode_mma_ctas_per_sm(int(head_dim), int(stages)))
        if per_sm <= 0:
            raise RuntimeError(f"decode attention kernel for head size {head_dim}: occupancy query failed")
        _decode_mma_resident[key] = per_sm * sm_count(device)
    return _decode_mma_resident[key]


def attention_decode_mma(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         token_pos: torch.Tensor, token_seq: torch.Tensor, page_table: torch.Tensor,
                         out: torch.Tensor, heads: int, kv_heads: int, head_dim: int, window: int,
                         scale: float, n_splits: int = 1, partial: Optional[torch.Tensor] = None,
                         tickets: Optional[torch.Tensor] = None, stages: int = 0) -> None:
    """Decode attention on the tensor cores (head sizes 64 and 128).  With several
    splits the slice that finishes last merges them: ``out`` is always complete.
    ``tickets``: int32 zeros, ``mma_ticket_count`` of them, left zero.  ``stages``:
    pages in flight per CTA (0: the default; fewer let more CTAs share an SM)."""
    _cuda(k_cache, v_cache, token_pos, token_seq, page_table, out, partial, tickets)
    _need(q.is_cuda and q.dtype == torch.bfloat16 == k_cache.dtype == out.dtype,
          "attention_decode_mma: bfloat16 tensors")
    n = out.shape[0]
    pages, nkv, page_size, d = k_cache.shape
    _need(nkv == kv_heads and d == head_dim, "cache shape differs from the heads given")
    _need(attention_decode_mma_takes(head_dim, page_size),
          f"attention_decode_mma: head_dim {head_dim} / page {page_size} is not taken")
    _need(heads % kv_heads == 0, "attention: heads is not a multiple of kv_heads")
    _need(pages * nkv * page_size < 2 ** 31, "attention: the cache has too many rows")
    _need(out.shape[1] == heads * head_dim and n <= 65535, "attention: out [n <= 65535, heads * d]")
    if n_splits > 1:
        _need(partial is not None and partial.dtype == torch.float32
              and partial.numel() >= n * heads * n_splits * (head_dim + 2),
              "attention: partial scratch too small")
        _need(tickets is not None and tickets.dtype == torch.int32
              and tickets.numel() >= mma_ticket_count(n, heads, kv_heads), "attention: tickets")
    _check(_lib().nnis_attention_decode_mma_staged(
        _ptr(q), q_stride, _ptr(k_cache), _ptr(v_cache), _ptr(token_pos), _ptr(token_seq),
        _ptr(page_table), page_table.shape[1], _ptr(out), _ptr(partial), _ptr(tickets), n, heads,
        kv_heads, head_dim, page_size, window, ctypes.c_float(scale), n_splits, int(stages), PDL,
        _stream()), "attention_decode_mma")


def attention_prefill_mma(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                          tiles: torch.Tensor, seq_first_row: torch.Tensor, seq_start: torch.Tensor,
                          seq_count: torch.Tensor, page_table: torch.Tensor, out: torch.Tensor,
                          heads: int, kv_heads: int, head_dim: int, window: int, scale: float) -> None:
    """Prompt attention on the tensor cores (head sizes 64 and 128): packed query
    tokens, 64 per tile, each over its own sequence's keys in the paged cache."""
    _cuda(k_cache, v_cache, tiles, seq_first_row, seq_start, seq_count, page_table, out)
    _need(q.is_cuda and q.dtype == torch.bfloat16 == k_cache.dtype == out.dtype,
          "attention_prefill_mma: bfloat16 tensors")
    pages, nkv, page_size, d = k_cache.shape
    _need(nkv == kv_heads and d == head_dim, "cache shape differs from the heads given")
    _need(attention_decode_mma_takes(head_dim, page_size),
          f"attention_prefill_mma: head_dim {head_dim} / page {page_size} is not taken")
    _need(heads % kv_heads == 0, "attention: heads is not a multiple of kv_heads")
    _need(pages * nkv * page_size < 2 ** 31, "attention: the cache has too many rows")
    _need(out.shape[1] == heads * head_dim, "attention: out [n, heads * d]")
    for t in (tiles, seq_first_row, seq_start, seq_count):
        _need(t.dtype == torch.int32, "attention_prefill_mma: int32 tables")
    _need(tiles.dim() == 2 and tiles.shape[1] == 2 and tiles.shape[0] > 0, "tiles: int32 [n_tiles, 2]")
    _check(_lib().nnis_attention_prefill_mma(
        _ptr(q), q_stride, _ptr(k_cache), _ptr(v_cache), _ptr(tiles), tiles.shape[0],
        _ptr(seq_first_row), _ptr(seq_start), _ptr(seq_count), _ptr(page_table), page_table.shape[1],
        _ptr(out), heads, kv_heads, head_dim, page_size, window, ctypes.c_float(scale), _stream()),
        "attention_prefill_mma")


WIDE_QUERY_TILE = 128  # queries per CTA of attention_prefill_tc
TC_ATTENTION = 0 if os.environ.get("NNIS_TC_ATTENTION", "1") == "0" else 1


def attention_prefill_tc_takes(head_dim: int, page_size: int, q_stride: int) -> bool:
    """Whether the tcgen05 prompt attention kernel runs these sizes."""
    return bool(TC_ATTENTION) and head_dim == 64 and page_size == 64 and q_stride % 8 == 0


def prefill_tc_plan(counts, starts, window: int, heads: int, sms: int):
    """Work list of attention_prefill_tc for a step whose sequences bring
    ``counts`` tokens after ``starts`` cached ones.

    A tile is 128 queries of one sequence; its keys are the pages from its first
    query's window start to its last query.  Two CTAs share an SM, so tiles are cut
    into chunks of pages while there would be fewer CTAs (units x heads) than 1.7
    per SM: the longest chunk of 32, 24, 16 or 12 pages that gives as many, else 8
    (a chunk costs a CTA's start and end, a trip of its rows through scratch and,
    for the last one of a tile, the merge; measured on one prompt of 1,024 / 2,048 /
    4,096 tokens and 9 heads the best lengths were 8 / 12 / none); then the shortest
    chunks from 8 pages on with which the CTAs still fit one wave of two to an SM (2,048
    tokens: 11 pages, 288 CTAs; a CTA walks its pages one after another).  Returns ``units`` int32 [n, 4] (sequence,
    first query, chunk | chunks << 16, first scratch slot), longest first, and the
    number of scratch slots.  ``prefill_tc_pays`` says whether the step is worth this
    kernel at all."""
    import numpy as np
    tiles = []
    for i, (c, st) in enumerate(zip(counts, starts)):
        for q0 in range(0, int(c), WIDE_QUERY_TILE):
            rows = min(WIDE_QUERY_TILE, int(c) - q0)
            pos0 = int(st) + q0
            lo = max(0, pos0 - window + 1) if window > 0 else 0
            tiles.append((i, q0, (pos0 + rows - 1) // 64 - lo // 64 + 1))
    chunk_pages = 8
    for cand in (1 << 30, 32, 24, 16, 12):
        if 10 * sum(-(-p // cand) for _, _, p in tiles) * heads >= 17 * sms:
            chunk_pages = cand
            break
    if PREFILL_SHORT_CHUNKS and chunk_pages > 8 and chunk_pages < (1 << 30):
        # A CTA walks its pages one after another (1.3 us a page): where the CTAs still fit
        # one wave of two to an SM with shorter chunks, the shortest such chunks end first.
        for cand in range(8, chunk_pages):
            if sum(-(-p // cand) for _, _, p in tiles) * heads <= 2 * sms:
                chunk_pages = cand
                break
    units, slot = [], 0
    for i, q0, pages in tiles:
        n = -(-pages // chunk_pages)
        while n > 1 and (n - 1) * (-(-pages // n)) >= pages:  # no chunk may be empty
            n -= 1
        per = -(-pages // n)
        for c in range(n):
            units.append((min(per, pages - c * per), i, q0, c | (n << 16), slot if n > 1 else 0))
        if n > 1:
            slot += n
    units.sort(key=lambda u: -u[0])
    return np.asarray([u[1:] for u in units], dtype=np.int32).reshape(-1, 4), slot


def prefill_tc_pays(counts, starts, window: int) -> bool:
    """Whether a step's tiles are long enough for attention_prefill_tc: with fewer
    than two and a half pages of keys per 128-query tile on average (many short
    prompts) the 64-query tiles of the mma.sync kernel waste less and run as fast
    or faster (8 x 128 tokens: 5.4 against 6.2 us; 8 x 256: 9.8 against 7.7 us)."""
    tiles = pages = 0
    for c, st in zip(counts, starts):
        for q0 in range(0, int(c), WIDE_QUERY_TILE):
            rows = min(WIDE_QUERY_TILE, int(c) - q0)
            pos0 = int(st) + q0
            lo = max(0, pos0 - window + 1) if window > 0 else 0
            tiles += 1
            pages += (pos0 + rows - 1) // 64 - lo // 64 + 1
    return tiles > 0 and 2 * pages >= 5 * tiles


PREFILL_TC_PARTIAL = 66 * WIDE_QUERY_TILE  # float32 per (scratch slot, head)


def attention_prefill_tc(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         units: torch.Tensor, partial: Optional[torch.Tensor],
                         tickets: Optional[torch.Tensor], seq_first_row: torch.Tensor,
                         seq_start: torch.Tensor, seq_count: torch.Tensor, page_table: torch.Tensor,
                         out: torch.Tensor, heads: int, kv_heads: int, head_dim: int, window: int,
                         scale: float) -> None:
    """Prompt attention on tcgen05 (head size 64): packed query tokens, each over
    its own sequence's keys in the paged cache.  ``units`` comes from
    ``prefill_tc_plan``; when it cuts tiles, ``partial`` is float32 scratch of
    slots x heads x PREFILL_TC_PARTIAL values and ``tickets`` int32 [slots x heads],
    zero before the first launch (the kernel leaves them zero)."""
    _cuda(k_cache, v_cache, units, seq_first_row, seq_start, seq_count, page_table, out)
    _need(q.is_cuda and q.dtype == torch.bfloat16 == k_cache.dtype == out.dtype,
          "attention_prefill_tc: bfloat16 tensors")
    pages, nkv, page_size, d = k_cache.shape
    _need(nkv == kv_heads and d == head_dim, "cache shape differs from the heads given")
    _need(attention_prefill_tc_takes(head_dim, page_size, q_stride),
          f"attention_prefill_tc: head_dim {head_dim} / page {page_size} / stride {q_stride} is not taken")
    _need(heads % kv_heads == 0, "attention: heads is not a multiple of kv_heads")
    _need(pages * nkv * page_size < 2 ** 31, "attention: the cache has too many rows")
    _need(out.shape[1] == heads * head_dim and out.is_contiguous(), "attention: out [n, heads * d]")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "attention: contiguous cache")
    for t in (units, seq_first_row, seq_start, seq_count):
        _need(t.dtype == torch.int32, "attention_prefill_tc: int32 tables")
    _need(units.dim() == 2 and units.shape[1] == 4 and units.shape[0] > 0 and units.is_contiguous(),
          "units: int32 [n_units, 4]")
    if partial is not None:
        _cuda(partial, tickets)
        _need(partial.dtype == torch.float32 and tickets.dtype == torch.int32,
              "partial: float32 scratch, tickets: int32")
    _check(_lib().nnis_attention_prefill_tc(
        _ptr(q), q_stride, out.shape[0], _ptr(k_cache), _ptr(v_cache),
        ctypes.c_longlong(pages * nkv * page_size), _ptr(units), units.shape[0],
        _ptr(partial) if partial is not None else None, _ptr(tickets) if partial is not None else None,
        _ptr(seq_first_row), _ptr(seq_start), _ptr(seq_count), _ptr(page_table), page_table.shape[1],
        _ptr(out), heads, kv_heads, head_dim, page_size, window, ctypes.c_float(scale),
        _ptr(status_word(out.device)), PDL, _stream()),
        "attention_prefill_tc")


def mma_ticket_count(n: int, heads: int, kv_heads: int) -> int:
    return n * kv_heads * (-(-(heads // kv_heads) // 16))


TC_GEMM = 0 if os.environ.get("NNIS_TC_GEMM", "1") == "0" else 1


def gemm_tc_takes(m: int, n: int, k: int) -> bool:
    """Whether the tcgen05 kernel runs this bfloat16 product (else CUDA cores):
    K a multiple of 8 (rows of 16 bytes for TMA) and enough rows to fill a tile."""
    return bool(TC_GEMM) and m > 16 and k % 8 == 0 and -(-m // 128) <= 65535


GEMM_GATED, GEMM_QKV = 3, 4


def gemm_tc(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
            mode: int, token_pos: Optional[torch.Tensor] = None,
            token_seq: Optional[torch.Tensor] = None, page_table: Optional[torch.Tensor] = None,
            cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
            k_cache: Optional[torch.Tensor] = None, v_cache: Optional[torch.Tensor] = None,
            heads: int = 0, kv_heads: int = 0, head_dim: int = 0, page_size: int = 0,
            split_scratch: Optional[torch.Tensor] = None,
            split_tickets: Optional[torch.Tensor] = None) -> None:
    """out (op)= a . w^T + bias on the tensor cores (tcgen05, float32 accumulation
    in tensor memory); bfloat16 operands.  Modes: STORE, STORE_F32, ADD_F32,
    GEMM_GATED (w = [gate; up] rows, out bfloat16 [m, n / 2] = silu(gate) * up) and
    GEMM_QKV (bias, RoPE at each row's position, q to out [m, heads * d], k and v
    into the paged cache; head_dim 64 or 128).  ADD_F32 with ``split_scratch`` (float32)
    and ``split_tickets`` (int32, zero; left zero) of the sizes ``gemm_tc_splits`` names
    may cut K among several CTAs per tile; their sums are added in a fixed order."""
    _cuda(a, w, bias, out, token_pos, token_seq, page_table, cos, sin, k_cache, v_cache)
    m, k = a.shape
    n = w.shape[0]
    _need(a.dtype == w.dtype == torch.bfloat16 and w.shape[1] == k, "gemm_tc: bfloat16 a [m, k], w [n, k]")
    _need(gemm_tc_takes(m, n, k), f"gemm_tc: shape m={m} n={n} k={k} is not taken")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n, "gemm_tc: bias float32 [n]")
    if mode == GEMM_GATED:
        _need(n % 2 == 0 and out.dtype == torch.bfloat16 and tuple(out.shape) == (m, n // 2),
              "gemm_tc: gated out bfloat16 [m, n / 2]")
    elif mode == GEMM_QKV:
        _need(gemm_tc_qkv_takes(head_dim) and n == (heads + 2 * kv_heads) * head_dim,
              "gemm_tc: qkv rows / head_dim not taken")
        _need(out.dtype == torch.bfloat16 and tuple(out.shape) == (m, heads * head_dim),
              "gemm_tc: q out bfloat16 [m, heads * d]")
        _need(token_pos is not None and token_pos.dtype == torch.int32 and token_pos.numel() >= m,
              "gemm_tc: token_pos int32 [m]")
        if kv_heads > 0:
            _need(k_cache is not None and k_cache.dtype == torch.bfloat16
                  and tuple(k_cache.shape[1:]) == (kv_heads, page_size, head_dim)
                  and page_table is not None and token_seq is not None, "gemm_tc: cache [pages, kv, page, d]")
        if cos is not None:
            _need(cos.dtype == torch.float32 and cos.shape[1] == head_dim // 2, "gemm_tc: cos/sin tables")
    else:
        _need(tuple(out.shape) == (m, n), "gemm_tc: out [m, n]")
        _need(out.dtype == (torch.bfloat16 if mode == STORE else torch.float32), "gemm_tc: out dtype vs mode")
    cols = page_table.shape[1] if page_table is not None else 0
    scratch, tickets = (split_scratch, split_tickets) if mode == ADD_F32 else (None, None)
    _cuda(scratch, tickets)
    _check(_lib().nnis_gemm_tc(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), m, n, k, mode, _ptr(token_pos),
                               _ptr(token_seq), _ptr(page_table), cols, _ptr(cos), _ptr(sin),
                               _ptr(k_cache), _ptr(v_cache), heads, kv_heads, head_dim, page_size,
                               _ptr(scratch), ctypes.c_longlong(scratch.numel() if scratch is not None else 0),
                               _ptr(tickets), tickets.numel() if tickets is not None else 0,
                               sm_count(a.device), _ptr(status_word(a.device)), PDL, _stream()),
           "gemm_tc")


# Whether the adding product may cut a long K among CTAs (few tiles): parts/linear.py asks.
def gemm_tc_glu_clamp(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                      limit: float, alpha: float) -> None:
    """The gated tensor-core product with the clamped activation in its epilogue: w = [gate; up] rows,
    out bfloat16 [m, n / 2] = g' sigmoid(alpha g') (u' + 1), g' = min(gate, limit), u' = up clamped to
    [-limit, limit]."""
    _cuda(a, w, bias, out)
    m, k = a.shape
    n = w.shape[0]
    _need(a.dtype == w.dtype == torch.bfloat16 and w.shape[1] == k, "gemm_tc_glu_clamp: bfloat16 a [m, k], w [n, k]")
    _need(gemm_tc_takes(m, n, k) and limit > 0, f"gemm_tc_glu_clamp: shape m={m} n={n} k={k} is not taken")
    _need(n % 2 == 0 and out.dtype == torch.bfloat16 and tuple(out.shape) == (m, n // 2),
          "gemm_tc_glu_clamp: out bfloat16 [m, n / 2]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n, "gemm_tc_glu_clamp: bias float32 [n]")
    _check(_lib().nnis_gemm_tc_glu_clamp(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), m, n, k, ctypes.c_float(limit),
                                         ctypes.c_float(alpha), sm_count(a.device), _ptr(status_word(a.device)),
                                         PDL, _stream()), "gemm_tc_glu_clamp")


def gemm_tc_act(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, act: int) -> None:
    """The storing tensor-core product with an activation in its epilogue: out bfloat16 [m, n] =
    act(a . w^T + bias); ``GEMM_ACT_RELU2``, ``GEMM_ACT_GELU_ERF`` or ``GEMM_ACT_GELU_TANH``."""
    _cuda(a, w, bias, out)
    m, k = a.shape
    n = w.shape[0]
    _need(a.dtype == w.dtype == torch.bfloat16 and w.shape[1] == k, "gemm_tc_act: bfloat16 a [m, k], w [n, k]")
    _need(gemm_tc_takes(m, n, k), f"gemm_tc_act: shape m={m} n={n} k={k} is not taken")
    _need(out.dtype == torch.bfloat16 and tuple(out.shape) == (m, n), "gemm_tc_act: out bfloat16 [m, n]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n, "gemm_tc_act: bias float32 [n]")
    _check(_lib().nnis_gemm_tc_act(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), m, n, k, act, sm_count(a.device),
                                   _ptr(status_word(a.device)), PDL, _stream()), "gemm_tc_act")


GEMM_SPLIT_K = os.environ.get("NNIS_GEMM_SPLIT_K", "1") == "1"


def gemm_tc_splits(m: int, n: int, k: int, device=None):
    """(CTAs that share a tile of the adding product, float32 of scratch, tickets)."""
    floats, tiles = ctypes.c_longlong(0), ctypes.c_int(0)
    sms = sm_count(device) if device is not None else 148
    splits = int(_lib().nnis_gemm_tc_splits(m, n, k, sms, ctypes.byref(floats), ctypes.byref(tiles)))
    return splits, int(floats.value), int(tiles.value)


def gemm_tc_qkv_takes(head_dim: int) -> bool:
    return head_dim in (64, 128)


def advance(tokens: torch.Tensor, pos: torch.Tensor, picked: torch.Tensor) -> None:
    """tokens = picked; pos += 1, on live rows (pos >= 0) only."""
    _cuda(tokens, pos, picked)
    _need(tokens.dtype == pos.dtype == picked.dtype == torch.int32, "advance: int32")
    n = tokens.numel()
    _need(pos.numel() == n and picked.numel() >= n, "advance: sizes differ")
    _check(_lib().nnis_advance(_ptr(tokens), _ptr(pos), _ptr(picked), n, _stream()), "advance")


# ---------------------------------------------------------------------------
# The timeline of a step (trace.cu), for measurements.
_trace_buffer: Optional[torch.Tensor] = None


def trace_begin(capacity: int = 2048, device="cuda:0") -> torch.Tensor:
    """From now on every launch of an instrumented kernel (decode projections, decode
    attention) takes a slot of the returned buffer, int64 [capacity, 8]: first CTA's
    begin, last CTA's end, first and last CTA past the wait for the kernel before, and
    first and last CTA at two marks inside the kernel, in nanoseconds of the GPU's timer.  A graph captured meanwhile keeps its slots."""
    global _trace_buffer
    _trace_buffer = torch.zeros((capacity, 8), dtype=torch.int64, device=device)
    trace_clear()
    _lib().nnis_trace_set(_ptr(_trace_buffer), capacity)
    return _trace_buffer


def trace_clear() -> None:
    """Before the replay that is to be read: earliest words to the largest value, latest to zero."""
    _trace_buffer[:, 0::2] = torch.iinfo(torch.int64).max
    _trace_buffer[:, 1::2] = 0


def trace_end():
    """Stops handing out slots; returns the names of the launches that took one."""
    lib = _lib()
    lib.nnis_trace_name.restype = ctypes.c_char_p
    names = [lib.nnis_trace_name(i).decode() for i in range(int(lib.nnis_trace_count()))]
    lib.nnis_trace_set(None, 0)
    return names


# ---------------------------------------------------------------------------
# norm in groups, per-head products, latent attention, retention, experts
# ---------------------------------------------------------------------------
# grouped products on the tensor cores (experts of prompt steps, per-head products of many rows)
MOE_GROUPED = 0 if os.environ.get("NNIS_MOE_GROUPED", "1") == "0" else 1

def group_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, groups: int, out: torch.Tensor,
                  rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = x[rows[r]] (or x[r]) with each of ``groups`` equal runs divided by its own
    root mean square, times weight; statistics in float32.  ``out`` may be ``x`` itself."""
    _cuda(x, weight, out, rows)
    n, width = out.shape
    _need(x.dtype == torch.float32 and x.shape[1] == width, "x: float32 [*, width]")
    _need(weight.dtype == torch.float32 and weight.numel() == width, "weight: float32 [width]")
    _need(groups > 0 and width % groups == 0, f"norm: {groups} groups do not divide the width {width}")
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.numel() >= n, "rows: int32 [n]")
    else:
        _need(x.shape[0] >= n, "x has fewer rows than out")
    _check(_lib().nnis_group_rmsnorm(_ptr(x), _ptr(rows), _ptr(weight), _ptr(out), code_of(out.dtype), n,
                                     width, groups, ctypes.c_float(eps), _stream()), "group_rmsnorm")


def add_rows(a: torch.Tensor, b: torch.Tensor) -> None:
    """a += b, float32 of equal shape (a count of values that is a multiple of four)."""
    _cuda(a, b)
    _need(a.dtype == b.dtype == torch.float32 and a.shape == b.shape and a.numel() % 4 == 0,
          "add_rows: float32 tensors of one shape, a multiple of four values")
    _check(_lib().nnis_add_rows(_ptr(a), _ptr(b), ctypes.c_longlong(a.numel()), _stream()), "add_rows")


def relu2_gate(u: torch.Tensor, out: torch.Tensor) -> None:
    """out = relu(u[:, :I])^2 for out [n, I]; when u has more columns than that, times
    sigmoid(u[:, I]) (the columns after the gate's are padding)."""
    _cuda(u, out)
    n, inter = out.shape
    _need(u.dtype == torch.float32 and u.shape[0] == n and u.shape[1] >= inter, "u: float32 [n, >= inter]")
    _check(_lib().nnis_relu2_gate(_ptr(u), _ptr(out), code_of(out.dtype), ctypes.c_longlong(n), inter,
                                  u.shape[1] - inter, _stream()), "relu2_gate")


def rope_part(src: torch.Tensor, src_head: int, src_off: int, dst: torch.Tensor, dst_head: int,
              dst_off: int, token_pos: torch.Tensor, freq: torch.Tensor, heads: int, length: int,
              dims: int) -> None:
    """For every row n and head h, the ``length`` elements at src[n, h * src_head + src_off]
    go to dst[n, h * dst_head + dst_off]; the first ``dims`` are turned in pairs (i, i +
    dims / 2) by the angle position * freq[i], the rest pass unchanged."""
    _cuda(src, dst, token_pos, freq)
    n = src.shape[0]
    _need(src.dtype == dst.dtype and dst.shape[0] == n, "rope_part: src and dst of one dtype and row count")
    _need(src_off + length <= src_head and (heads - 1) * src_head + src_off + length <= src.shape[1],
          "rope_part: the part lies outside src's heads")
    _need(dst_off + length <= dst_head and (heads - 1) * dst_head + dst_off + length <= dst.shape[1],
          "rope_part: the part lies outside dst's heads")
    _need(freq.dtype == torch.float32 and freq.numel() >= dims // 2 and dims % 2 == 0 and dims <= length,
          "rope_part: freq float32 [dims / 2]")
    _need(token_pos.dtype == torch.int32 and token_pos.numel() >= n, "rope_part: token_pos int32 [n]")
    _check(_lib().nnis_rope_part(_ptr(src), ctypes.c_longlong(src.shape[1]), src_head, src_off, _ptr(dst),
                                 ctypes.c_longlong(dst.shape[1]), dst_head, dst_off, _ptr(token_pos),
                                 _ptr(freq), n, heads, length, dims, code_of(src.dtype), _stream()),
           "rope_part")


def batched_linear(a: torch.Tensor, a_head: int, w: torch.Tensor, out: torch.Tensor, out_head: int) -> None:
    """out[m, b * out_head : + N] = a[m, b * a_head : + K] . w[b]^T for every head b;
    w [heads, N, K]; a and out packed rows whose heads are ``a_head`` / ``out_head`` apart."""
    _cuda(a, w, out)
    heads, n, k = w.shape
    m = a.shape[0]
    _need(a.dtype == w.dtype == out.dtype and out.shape[0] == m, "batched_linear: one dtype, equal rows")
    _need(k <= a_head and (heads - 1) * a_head + k <= a.shape[1], "batched_linear: K lies outside a's heads")
    _need(n <= out_head and (heads - 1) * out_head + n <= out.shape[1],
          "batched_linear: N lies outside out's heads")
    if a.dtype == torch.bfloat16 and m > 16 and MOE_GROUPED and k % 8 == 0 and a.shape[1] % 8 == 0 \
            and a_head % 8 == 0:
        # many rows: 64 x 64 tiles on the tensor cores (the grouped products' kernel)
        _check(_lib().nnis_batched_linear_mma(_ptr(a), ctypes.c_longlong(a.shape[1]), ctypes.c_longlong(a_head),
                                              _ptr(w), _ptr(out), ctypes.c_longlong(out.shape[1]),
                                              ctypes.c_longlong(out_head), heads, m, n, k, _stream()),
               "batched_linear_mma")
        return
    _check(_lib().nnis_batched_linear(_ptr(a), ctypes.c_longlong(a.shape[1]), ctypes.c_longlong(a_head),
                                      _ptr(w), _ptr(out), ctypes.c_longlong(out.shape[1]),
                                      ctypes.c_longlong(out_head), heads, m, n, k, code_of(a.dtype),
                                      _stream()), "batched_linear")


def latent_prep(a: torch.Tensor, wq: torch.Tensor, wkv: torch.Tensor, freq: torch.Tensor,
                token_pos: torch.Tensor, token_seq: torch.Tensor, page_table: torch.Tensor,
                cq: torch.Tensor, cache: torch.Tensor, q_rank: int, kv_rank: int, rot: int,
                rot_dims: int, eps: float) -> None:
    """From the down-projection's float32 rows [q latent | c raw | kr raw]: the normed q
    latent to ``cq``; the normed c and the rotated kr into the cache row of each token."""
    _cuda(a, wq, wkv, freq, token_pos, token_seq, page_table, cq, cache)
    n = a.shape[0]
    _need(a.dtype == torch.float32 and a.shape[1] == q_rank + kv_rank + rot, "latent_prep: a float32 rows")
    _need(wq.dtype == wkv.dtype == freq.dtype == torch.float32 and wq.numel() == q_rank
          and wkv.numel() == kv_rank and freq.numel() >= rot_dims // 2, "latent_prep: float32 vectors")
    _need(cq.dtype == cache.dtype and tuple(cq.shape) == (n, q_rank), "latent_prep: cq [n, q_rank]")
    _need(cache.dim() == 4 and cache.shape[1] == 1 and cache.shape[3] == kv_rank + rot,
          "latent_prep: cache [pages, 1, page, kv_rank + rot]")
    _need(page_table.dtype == torch.int32 and token_pos.dtype == torch.int32, "latent_prep: int32 tables")
    _check(_lib().nnis_latent_prep(_ptr(a), _ptr(wq), _ptr(wkv), _ptr(freq), _ptr(token_pos),
                                   _ptr(token_seq), _ptr(page_table), page_table.shape[1], _ptr(cq),
                                   _ptr(cache), n, q_rank, kv_rank, rot, rot_dims, cache.shape[2],
                                   ctypes.c_float(eps), code_of(cq.dtype), _stream()), "latent_prep")


def attention_latent(q: torch.Tensor, cache: torch.Tensor, token_pos: torch.Tensor,
                     token_seq: torch.Tensor, page_table: torch.Tensor, out: torch.Tensor, heads: int,
                     dv: int, scale: float, n_splits: int = 1,
                     partial: Optional[torch.Tensor] = None) -> None:
    """Causal attention of packed queries [n, heads * dk] over cache rows [pages, 1, page,
    dk] shared by all heads; the rows' first ``dv`` values are the values.  out [n, heads * dv]."""
    _cuda(q, cache, token_pos, token_seq, page_table, out, partial)
    n = out.shape[0]
    pages, one, page_size, dk = cache.shape
    _need(one == 1 and q.shape[1] == heads * dk and out.shape[1] == heads * dv and 0 < dv <= dk,
          "attention_latent: q [n, heads * dk], out [n, heads * dv]")
    _need(q.dtype == cache.dtype == out.dtype, "attention_latent: one dtype")
    _need(pages * page_size < 2 ** 31, "attention_latent: the cache has too many rows")
    if n_splits > 1:
        _need(partial is not None and partial.dtype == torch.float32
              and partial.numel() >= n * heads * n_splits * (dv + 2), "attention_latent: partial scratch")
    _check(_lib().nnis_attention_latent(_ptr(q), _ptr(cache), _ptr(token_pos), _ptr(token_seq),
                                        _ptr(page_table), page_table.shape[1], _ptr(out), _ptr(partial), n,
                                        heads, dk, dv, page_size, ctypes.c_float(scale), n_splits,
                                        code_of(out.dtype), _stream()),
           "attention_latent", 2 if n_splits > 1 else 1)


def retention(qkvg: torch.Tensor, freq: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
              token_pos: torch.Tensor, token_seq: torch.Tensor, seq_slots: torch.Tensor,
              seq_first_row: Optional[torch.Tensor], seq_start: Optional[torch.Tensor],
              seq_count: Optional[torch.Tensor], o_raw: torch.Tensor, out: torch.Tensor, heads: int,
              dim: int, vdim: int, rot_dims: int, eps: float, segments: Optional[torch.Tensor] = None,
              seq_first_segment: Optional[torch.Tensor] = None, seg_state: Optional[torch.Tensor] = None,
              seg_len: int = 0, activation: bool = False, key_scale: Optional[float] = None,
              norm_weight: Optional[torch.Tensor] = None, gate: str = "silu") -> None:
    """Retention of packed rows [q | k | v | g] from and into the per-slot state
    [slots, heads, dim, vdim] (float32); out [n, heads * vdim] = o / rms(o) * silu(g).
    ``activation``: q, k and v pass silu as they are read; ``key_scale``: what multiplies k
    (dim^-1/2 unless given); ``norm_weight`` (float32 [heads * vdim]): one norm over a token's
    joined heads, times this weight, instead of a norm per head; ``gate``: "silu" or "sigmoid".
    Without ``seq_first_row`` every row is one token of a sequence of its own.  With
    ``segments`` (``retention_segments``) a prompt step's sequences are cut into runs of
    ``seg_len`` tokens that are worked side by side (``retention_takes_segments``)."""
    _cuda(qkvg, freq, decay, state, token_pos, token_seq, seq_slots, seq_first_row, seq_start, seq_count,
          o_raw, out, segments, seq_first_segment, seg_state, norm_weight)
    _need(gate in ("silu", "sigmoid"), "retention: the gate is silu or sigmoid")
    _need(norm_weight is None or (norm_weight.dtype == torch.float32 and norm_weight.numel() == heads * vdim),
          "retention: norm_weight float32 [heads * vdim]")
    n_segments = 0
    if segments is not None:
        n_segments = segments.shape[0]
        _need(retention_takes_segments(dim) and seq_first_row is not None and seq_first_segment is not None
              and seg_state is not None and seg_state.dtype == torch.float32
              and seg_state.numel() >= n_segments * heads * dim * vdim and seg_len > 0,
              "retention: segments need a prompt step, their tables and scratch")
    n = out.shape[0]
    _need(qkvg.shape[0] >= n and qkvg.shape[1] == 2 * heads * (dim + vdim) and qkvg.dtype == out.dtype,
          "retention: rows [n, 2 heads (dim + vdim)]")
    _need(state.dtype == torch.float32 and tuple(state.shape[1:]) == (heads, dim, vdim),
          "retention: state float32 [slots, heads, dim, vdim]")
    _need(decay.dtype == torch.float32 and decay.numel() == heads and freq.dtype == torch.float32
          and freq.numel() >= rot_dims // 2, "retention: decay [heads], freq [rot_dims / 2] float32")
    _need(o_raw.dtype == torch.float32 and o_raw.numel() >= n * heads * vdim, "retention: scratch")
    _need(out.shape[1] == heads * vdim, "retention: out [n, heads * vdim]")
    units = seq_first_row.numel() if seq_first_row is not None else n
    _check(_lib().nnis_retention(_ptr(qkvg), _ptr(freq), _ptr(decay), _ptr(state), _ptr(token_pos),
                                 _ptr(token_seq), _ptr(seq_slots), _ptr(seq_first_row), _ptr(seq_start),
                                 _ptr(seq_count), _ptr(segments), n_segments, _ptr(seq_first_segment), seg_len,
                                 _ptr(seg_state), _ptr(o_raw), _ptr(out), n, units, heads, dim, vdim,
                                 rot_dims, ctypes.c_float(eps), 1 if activation else 0,
                                 ctypes.c_float(dim ** -0.5 if key_scale is None else key_scale),
                                 _ptr(norm_weight), 1 if gate == "sigmoid" else 0, code_of(out.dtype), _stream()),
           "retention", 4 if segments is not None else 2)


RETENTION_SEGMENT = int(os.environ.get("NNIS_RETENTION_SEGMENT", "256"))  # tokens of a run; 0: no runs


def retention_takes_segments(dim: int) -> bool:
    """Whether prompts of these key sizes can be cut into runs worked side by side."""
    return RETENTION_SEGMENT > 0 and RETENTION_SEGMENT % 32 == 0 and dim in (32, 64, 128, 256)


def retention_segments(counts, seg_len: int):
    """(segments [n, 2] = (sequence, first token of the run), first segment of every
    sequence [sequences + 1]) for a prompt step whose sequences bring ``counts`` tokens."""
    import numpy as np
    segments, first = [], [0]
    for i, c in enumerate(counts):
        segments += [(i, t) for t in range(0, int(c), seg_len)]
        first.append(len(segments))
    return np.asarray(segments, dtype=np.int32).reshape(-1, 2), np.asarray(first, dtype=np.int32)


def moe_route(h: torch.Tensor, w_router: torch.Tensor, b_router: Optional[torch.Tensor],
              token_pos: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, top: int,
              sigmoid_scores: bool = False) -> None:
    """ids, weights [n, top]: the ``top`` experts with the largest float32 logits
    w_router . h + b_router and the softmax over their logits; with ``sigmoid_scores`` the
    weights are the sigmoid of each chosen logit, not renormalised."""
    _cuda(h, w_router, b_router, token_pos, ids, weights)
    n, width = h.shape
    experts = w_router.shape[0]
    _need(w_router.dtype == torch.float32 and w_router.shape[1] == width, "moe_route: router float32 [E, width]")
    _need(b_router is None or (b_router.dtype == torch.float32 and b_router.numel() == experts),
          "moe_route: bias float32 [E]")
    _need(ids.dtype == torch.int32 and weights.dtype == torch.float32 and ids.numel() >= n * top
          and weights.numel() >= n * top and 0 < top <= experts, "moe_route: ids int32, weights float32 [n, top]")
    _check(_lib().nnis_moe_route(_ptr(h), _ptr(w_router), _ptr(b_router), _ptr(token_pos), _ptr(ids),
                                 _ptr(weights), n, width, experts, top, 1 if sigmoid_scores else 0,
                                 code_of(h.dtype), _stream()),
           "moe_route")


def moe_experts(h: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor,
                weights: torch.Tensor, token_pos: torch.Tensor, act: torch.Tensor,
                residual: torch.Tensor, top: int) -> None:
    """residual[n] += sum over the chosen experts of weight * W_down[e] relu(W_up[e] h[n])^2."""
    _cuda(h, w_up, w_down, ids, weights, token_pos, act, residual)
    n, width = h.shape
    experts, ff, _ = w_up.shape
    _need(tuple(w_up.shape) == (experts, ff, width) and tuple(w_down.shape) == (experts, width, ff)
          and h.dtype == w_up.dtype == w_down.dtype == act.dtype, "moe_experts: stacked weights of one dtype")
    _need(act.numel() >= n * top * ff, "moe_experts: act scratch [n, top, ff]")
    _need(residual.dtype == torch.float32 and tuple(residual.shape) == (n, width), "moe_experts: residual")
    _check(_lib().nnis_moe_experts(_ptr(h), _ptr(w_up), _ptr(w_down), _ptr(ids), _ptr(weights),
                                   _ptr(token_pos), _ptr(act), _ptr(residual), n, width, ff, top,
                                   code_of(h.dtype), _stream()), "moe_experts", 2)


LATENT_MMA = 0 if os.environ.get("NNIS_LATENT_MMA", "1") == "0" else 1


def latent_tile_rows(dv: int) -> int:
    """Stacked (token, head) rows per CTA of ``attention_latent_mma`` for output rows of dv values."""
    return int(_lib().nnis_attention_latent_mma_tile_rows(dv))


def attention_latent_mma_takes(dk: int, dv: int, page_size: int) -> bool:
    """Whether the tensor-core latent attention runs these sizes (bfloat16 only)."""
    return bool(LATENT_MMA) and bool(_lib().nnis_attention_latent_mma_takes(dk, dv, page_size))


def latent_tiles(counts, starts, heads: int, tile_rows: int):
    """The work list of ``attention_latent_mma`` for a prompt step: (sequence, first stacked
    row) per ``tile_rows`` rows of each sequence's tokens * heads rows, the tiles with the most
    pages to walk first (a causal prompt's last tiles are its longest: begun last they would
    run alone)."""
    import numpy as np
    tiles = [(i, r0) for i, c in enumerate(counts) for r0 in range(0, int(c) * heads, tile_rows)]
    tiles.sort(key=lambda t: -(int(starts[t[0]]) + (t[1] + tile_rows - 1) // heads))
    return np.asarray(tiles, dtype=np.int32).reshape(-1, 2)


def attention_latent_mma(q: torch.Tensor, cache: torch.Tensor, tiles: Optional[torch.Tensor],
                         seq_first_row: Optional[torch.Tensor], seq_start: Optional[torch.Tensor],
                         seq_count: Optional[torch.Tensor], token_pos: torch.Tensor, token_seq: torch.Tensor,
                         page_table: torch.Tensor, out: torch.Tensor, heads: int, dv: int, scale: float,
                         n_splits: int = 1, partial: Optional[torch.Tensor] = None) -> None:
    """``attention_latent`` on the tensor cores (bfloat16).  With ``tiles`` (``latent_tiles``) a
    prompt step; without, every row is one token of a sequence of its own."""
    _cuda(q, cache, tiles, seq_first_row, seq_start, seq_count, token_pos, token_seq, page_table, out, partial)
    n = out.shape[0]
    pages, one, page_size, dk = cache.shape
    _need(q.dtype == cache.dtype == out.dtype == torch.bfloat16, "attention_latent_mma: bfloat16")
    _need(one == 1 and q.shape[1] == heads * dk and out.shape[1] == heads * dv, "attention_latent_mma: shapes")
    _need(attention_latent_mma_takes(dk, dv, page_size), "attention_latent_mma: sizes not taken")
    _need(pages * page_size < 2 ** 31, "attention_latent_mma: the cache has too many rows")
    if n_splits > 1:
        _need(partial is not None and partial.dtype == torch.float32
              and partial.numel() >= n * heads * n_splits * (dv + 2), "attention_latent_mma: partial scratch")
    _check(_lib().nnis_attention_latent_mma(
        _ptr(q), _ptr(cache), _ptr(tiles), tiles.shape[0] if tiles is not None else 0, _ptr(seq_first_row),
        _ptr(seq_start), _ptr(seq_count), _ptr(token_pos), _ptr(token_seq), _ptr(page_table),
        page_table.shape[1], _ptr(out), _ptr(partial), n, heads, dk, dv, page_size, ctypes.c_float(scale),
        n_splits, _stream()), "attention_latent_mma", 2 if n_splits > 1 else 1)




def moe_grouped_takes(width: int, ff: int, experts: int) -> bool:
    """Whether the grouped tensor-core products run these sizes (bfloat16, prompt steps)."""
    return bool(MOE_GROUPED) and bool(_lib().nnis_moe_grouped_takes(width, ff, experts))


def moe_grouped_tiles(n_pairs: int, experts: int) -> int:
    return int(_lib().nnis_moe_grouped_tiles(ctypes.c_longlong(n_pairs), experts))


def moe_grouped(h: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor,
                weights: torch.Tensor, perm: torch.Tensor, place: torch.Tensor, tile_expert: torch.Tensor,
                act: torch.Tensor, y: torch.Tensor, residual: torch.Tensor, top: int) -> None:
    """``moe_experts`` for many tokens: pairs sorted by expert, two grouped products on the
    tensor cores, the chosen experts' outputs added in the router's order.  Every row of
    ``h`` is a token (no padding rows).  Scratch sizes: see ``moe_grouped_tiles``."""
    _cuda(h, w_up, w_down, ids, weights, perm, place, tile_expert, act, y, residual)
    n, width = h.shape
    experts, ff, _ = w_up.shape
    tiles = moe_grouped_tiles(n * top, experts)
    _need(h.dtype == w_up.dtype == w_down.dtype == act.dtype == torch.bfloat16, "moe_grouped: bfloat16")
    _need(tuple(w_up.shape) == (experts, ff, width) and tuple(w_down.shape) == (experts, width, ff),
          "moe_grouped: stacked weights")
    _need(moe_grouped_takes(width, ff, experts), "moe_grouped: sizes not taken")
    _need(perm.dtype == place.dtype == tile_expert.dtype == ids.dtype == torch.int32
          and perm.numel() >= tiles * 64 and place.numel() >= n * top and tile_expert.numel() >= tiles,
          "moe_grouped: int32 scratch")
    _need(act.numel() >= tiles * 64 * ff and y.dtype == torch.float32 and y.numel() >= tiles * 64 * width,
          "moe_grouped: act and y scratch")
    _need(residual.dtype == torch.float32 and tuple(residual.shape) == (n, width), "moe_grouped: residual")
    _check(_lib().nnis_moe_grouped(_ptr(h), _ptr(w_up), _ptr(w_down), _ptr(ids), _ptr(weights), _ptr(perm),
                                   _ptr(place), _ptr(tile_expert), _ptr(act), _ptr(y), _ptr(residual), n, width,
                                   ff, experts, top, _stream()), "moe_grouped", 4)


def moe_grouped_tc_tiles(n_pairs: int, experts: int) -> int:
    return int(_lib().nnis_moe_grouped_tiles_tc(ctypes.c_longlong(n_pairs), experts))


def moe_grouped_tc(h: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor,
                   weights: torch.Tensor, perm: torch.Tensor, place: torch.Tensor, tile_expert: torch.Tensor,
                   x_sorted: torch.Tensor, act: torch.Tensor, y: torch.Tensor,
                   residual: torch.Tensor, top: int) -> None:
    """``moe_grouped`` with both products on the tcgen05 kernel: runs padded to tiles of 128
    rows (``moe_grouped_tc_tiles``), the rows gathered into ``x_sorted`` [tiles * 128, width]
    first, relu^2 in the first product's epilogue."""
    _cuda(h, w_up, w_down, ids, weights, perm, place, tile_expert, x_sorted, act, y, residual)
    n, width = h.shape
    experts, ff, _ = w_up.shape
    rows = moe_grouped_tc_tiles(n * top, experts) * 128
    _need(h.dtype == w_up.dtype == w_down.dtype == act.dtype == x_sorted.dtype == torch.bfloat16,
          "moe_grouped_tc: bfloat16")
    _need(tuple(w_up.shape) == (experts, ff, width) and tuple(w_down.shape) == (experts, width, ff),
          "moe_grouped_tc: stacked weights")
    _need(moe_grouped_takes(width, ff, experts) and TC_GEMM, "moe_grouped_tc: sizes not taken")
    _need(perm.dtype == place.dtype == tile_expert.dtype == ids.dtype == torch.int32 and perm.numel() >= rows
          and place.numel() >= n * top and tile_expert.numel() >= rows // 128, "moe_grouped_tc: int32 scratch")
    _need(x_sorted.numel() >= rows * width and act.numel() >= rows * ff and y.dtype == torch.float32
          and y.numel() >= rows * width, "moe_grouped_tc: scratch")
    _need(residual.dtype == torch.float32 and tuple(residual.shape) == (n, width), "moe_grouped_tc: residual")
    _check(_lib().nnis_moe_grouped_tc(_ptr(h), _ptr(w_up), _ptr(w_down), _ptr(ids), _ptr(weights), _ptr(perm),
                                      _ptr(place), _ptr(tile_expert), _ptr(x_sorted), _ptr(act), _ptr(y),
                                      _ptr(residual), n, width, ff, experts, top, sm_count(h.device),
                                      _ptr(status_word(h.device)), PDL, _stream()), "moe_grouped_tc", 5)


# ---------------------------------------------------------------------------
# a norm on a sub-layer's output, activations, WKV, selective scan, attention with a sink
def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x (float32) in out's dtype, rounded once."""
    _cuda(x, out)
    _need(x.dtype == torch.float32 and x.numel() == out.numel(), "cast_rows: float32 in, as many values out")
    _check(_lib().nnis_cast_rows(_ptr(x), _ptr(out), code_of(out.dtype), ctypes.c_longlong(x.numel()),
                                 _stream()), "cast_rows")


def norm_scale_add(branch: torch.Tensor, weight: torch.Tensor, eps: float, mult: float,
                   hidden: torch.Tensor, out: Optional[torch.Tensor] = None, clear: bool = False) -> None:
    """hidden += mult * rmsnorm(branch) * weight (all float32); ``out``, if given, receives the
    new rows of hidden in its own dtype; with ``clear`` the rows of ``branch`` are zero afterwards."""
    _cuda(branch, weight, hidden, out)
    n, width = hidden.shape
    _need(branch.dtype == hidden.dtype == weight.dtype == torch.float32 and tuple(branch.shape) == (n, width)
          and weight.numel() == width, "norm_scale_add: float32 [n, width] rows and [width] weights")
    _need(out is None or tuple(out.shape) == (n, width), "norm_scale_add: out [n, width]")
    _check(_lib().nnis_norm_scale_add(_ptr(branch), _ptr(weight), _ptr(hidden), _ptr(out),
                                      code_of(out.dtype) if out is not None else F32, n, width,
                                      ctypes.c_float(eps), ctypes.c_float(mult), 1 if clear else 0, _stream()),
           "norm_scale_add")


def sandwich_close(branch: torch.Tensor, weight: torch.Tensor, eps: float, hidden: torch.Tensor,
                   history: Optional[torch.Tensor] = None, mix_weights: Optional[torch.Tensor] = None, terms: int = 0,
                   next_weight: Optional[torch.Tensor] = None, next_eps: float = 0.0,
                   normed: Optional[torch.Tensor] = None) -> None:
    """hidden += rmsnorm(branch) * weight and branch is zero afterwards (float32 [n, width]).  With
    ``terms`` > 0 the new rows are kept as history[terms - 1] and hidden becomes sum over j < terms of
    mix_weights[j] * history[j] (history float32 [at least terms, n, width]).  With ``next_weight``
    the RMS norm of the rows that hidden then holds, times next_weight, is written to ``normed``
    ([n, width], its own dtype)."""
    _cuda(branch, weight, hidden, history, mix_weights, next_weight, normed)
    n, width = hidden.shape
    _need(branch.dtype == hidden.dtype == weight.dtype == torch.float32 and tuple(branch.shape) == (n, width)
          and weight.numel() == width and hidden.is_contiguous() and branch.is_contiguous(),
          "sandwich_close: float32 [n, width] rows and [width] weights")
    if terms > 0:
        _need(history is not None and mix_weights is not None and history.dtype == mix_weights.dtype == torch.float32
              and history.dim() == 3 and history.shape[0] >= terms and tuple(history.shape[1:]) == (n, width)
              and history.is_contiguous() and mix_weights.numel() == terms,
              "sandwich_close: history [terms, n, width] and a weight per term")
    _need((next_weight is None) == (normed is None), "sandwich_close: next_weight and normed go together")
    if normed is not None:
        _need(next_weight.dtype == torch.float32 and next_weight.numel() == width and tuple(normed.shape) == (n, width)
              and normed.is_contiguous(), "sandwich_close: normed [n, width], float32 weights")
    _check(_lib().nnis_sandwich_close(_ptr(branch), _ptr(weight), ctypes.c_float(eps), _ptr(hidden),
                                      _ptr(history) if terms > 0 else None, _ptr(mix_weights) if terms > 0 else None,
                                      int(terms), _ptr(next_weight), ctypes.c_float(next_eps), _ptr(normed),
                                      code_of(normed.dtype) if normed is not None else F32, n, width, _stream()),
           "sandwich_close")


def glu_clamp(gate_up: torch.Tensor, out: torch.Tensor, limit: float, alpha: float) -> None:
    """out = g' * sigmoid(alpha * g') * (u' + 1) with g' = min(gate, limit) and u' = up clamped
    to [-limit, limit]; gate_up float32 [n, 2I] (gate columns first)."""
    _cuda(gate_up, out)
    n, inter = out.shape
    _need(gate_up.dtype == torch.float32 and tuple(gate_up.shape) == (n, 2 * inter),
          "glu_clamp: gate_up float32 [n, 2 * inter]")
    _check(_lib().nnis_glu_clamp(_ptr(gate_up), _ptr(out), code_of(out.dtype), ctypes.c_longlong(n), inter,
                                 ctypes.c_float(limit), ctypes.c_float(alpha), _stream()), "glu_clamp")


def tanh_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(x, out)
    _need(x.dtype == torch.float32 and x.numel() == out.numel(), "tanh_rows: float32 in, as many values out")
    _check(_lib().nnis_tanh_rows(_ptr(x), _ptr(out), code_of(out.dtype), ctypes.c_longlong(x.numel()),
                                 _stream()), "tanh_rows")


def softcap_rows(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap), float32 in place."""
    _cuda(x)
    _need(x.dtype == torch.float32 and cap > 0, "softcap_rows: float32 rows, a positive cap")
    if x.numel():
        _check(_lib().nnis_softcap_rows(_ptr(x), ctypes.c_longlong(x.numel()), ctypes.c_float(cap), _stream()),
               "softcap_rows")


def _seq_tables(token_pos, token_seq, seq_slots, seq_first_row, seq_count):
    _cuda(token_pos, token_seq, seq_slots, seq_first_row, seq_count)
    for t in (token_pos, token_seq, seq_slots, seq_first_row, seq_count):
        _need(t is None or t.dtype == torch.int32, "step tables: int32")
    _need((seq_first_row is None) == (seq_count is None), "seq_first_row and seq_count come together")


def wkv_mix(x: torch.Tensor, mu: torch.Tensor, prev: torch.Tensor, token_pos: torch.Tensor,
            token_seq: torch.Tensor, seq_slots: torch.Tensor, seq_first_row: Optional[torch.Tensor],
            seq_count: Optional[torch.Tensor], mixes: torch.Tensor) -> None:
    """mixes[s, n] = x[n] + (x'[n] - x[n]) * mu[s], x' the row of the token before (the row above,
    or ``prev[slot]`` for a step's first token of a sequence)."""
    _cuda(x, mu, prev, mixes)
    _seq_tables(token_pos, token_seq, seq_slots, seq_first_row, seq_count)
    n, width = x.shape
    streams = mu.shape[0]
    _need(mu.dtype == prev.dtype == torch.float32 and mu.shape[1] == width and prev.shape[1] == width,
          "wkv_mix: mu [streams, width], prev [slots, width] float32")
    _need(mixes.dtype == x.dtype and tuple(mixes.shape) == (streams, n, width), "wkv_mix: mixes [streams, n, width]")
    _check(_lib().nnis_wkv_mix(_ptr(x), _ptr(mu), _ptr(prev), _ptr(token_pos), _ptr(token_seq), _ptr(seq_slots),
                               _ptr(seq_first_row), _ptr(seq_count), _ptr(mixes), n, width, streams,
                               code_of(x.dtype), _stream()), "wkv_mix")


def wkv_scan(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, d: torch.Tensor, u: torch.Tensor,
             state: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor, seq_slots: torch.Tensor,
             seq_first_row: Optional[torch.Tensor], seq_count: Optional[torch.Tensor], o_raw: torch.Tensor,
             heads: int, dim: int, segments: Optional[torch.Tensor] = None,
             seq_first_segment: Optional[torch.Tensor] = None, seg_len: int = 0,
             seg_state: Optional[torch.Tensor] = None, seg_logw: Optional[torch.Tensor] = None) -> None:
    """The recurrence over the step's tokens, from and into ``state`` [slots, heads, dim, dim].  With
    ``segments`` (``scan_segments``) a prompt step's sequences are cut into runs of ``seg_len`` tokens that
    are worked side by side; scratch ``seg_state`` float32 [runs, heads, dim, dim], ``seg_logw`` [runs, heads, dim]."""
    _cuda(r, k, v, d, u, state, o_raw, segments, seq_first_segment, seg_state, seg_logw)
    _seq_tables(token_pos, token_seq, seq_slots, seq_first_row, seq_count)
    n = r.shape[0]
    _need(r.dtype == k.dtype == v.dtype and tuple(r.shape) == tuple(k.shape) == tuple(v.shape) == (n, heads * dim),
          "wkv_scan: r, k, v [n, heads * dim] of one dtype")
    _need(d.dtype == u.dtype == state.dtype == o_raw.dtype == torch.float32 and d.numel() == n * heads * dim
          and u.numel() == heads * dim and o_raw.numel() >= n * heads * dim
          and tuple(state.shape[1:]) == (heads, dim, dim), "wkv_scan: float32 decay rows, bonus, state, output")
    _need(dim <= 256, f"wkv_scan: heads of {dim} channels (at most 256)")
    units = seq_first_row.numel() if seq_first_row is not None else n
    n_segments = 0
    if segments is not None:
        n_segments = segments.shape[0]
        _need(seq_first_row is not None and seq_first_segment is not None and seg_len > 0
              and seg_state is not None and seg_state.dtype == torch.float32
              and seg_state.numel() >= n_segments * heads * dim * dim and seg_logw is not None
              and seg_logw.dtype == torch.float32 and seg_logw.numel() >= n_segments * heads * dim
              and segments.dtype == seq_first_segment.dtype == torch.int32,
              "wkv_scan: runs need a prompt step, their tables and scratch")
    _check(_lib().nnis_wkv_scan(_ptr(r), _ptr(k), _ptr(v), _ptr(d), _ptr(u), _ptr(state), _ptr(token_pos),
                                _ptr(token_seq), _ptr(seq_slots), _ptr(seq_first_row), _ptr(seq_count),
                                _ptr(segments), n_segments, _ptr(seq_first_segment), seg_len, _ptr(seg_state),
                                _ptr(seg_logw), _ptr(o_raw), units, heads, dim, code_of(r.dtype), _stream()),
           "wkv_scan", 3 if segments is not None else 1)


def wkv_finish(o_raw: torch.Tensor, gate: torch.Tensor, norm_w: torch.Tensor, x: torch.Tensor,
               prev: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor, seq_slots: torch.Tensor,
               seq_first_row: Optional[torch.Tensor], seq_count: Optional[torch.Tensor], out: torch.Tensor,
               heads: int, dim: int, eps: float) -> None:
    """out = o / rms(o) per head * norm_w * silu(gate); prev[slot] = the step's last row of x."""
    _cuda(o_raw, gate, norm_w, x, prev, out)
    _seq_tables(token_pos, token_seq, seq_slots, seq_first_row, seq_count)
    n, width = x.shape
    _need(gate.dtype == out.dtype == x.dtype and tuple(gate.shape) == tuple(out.shape) == (n, heads * dim),
          "wkv_finish: gate, out [n, heads * dim]")
    _need(o_raw.dtype == norm_w.dtype == prev.dtype == torch.float32 and norm_w.numel() == heads * dim
          and prev.shape[1] == width, "wkv_finish: float32 o_raw, norm weights, prev [slots, width]")
    _check(_lib().nnis_wkv_finish(_ptr(o_raw), _ptr(gate), _ptr(norm_w), _ptr(x), _ptr(prev), _ptr(token_pos),
                                  _ptr(token_seq), _ptr(seq_slots), _ptr(seq_first_row), _ptr(seq_count),
                                  _ptr(out), n, heads, dim, width, ctypes.c_float(eps), code_of(x.dtype),
                                  _stream()), "wkv_finish")


def conv_silu(xz: torch.Tensor, conv_w: torch.Tensor, conv_b: Optional[torch.Tensor], conv_state: torch.Tensor,
              token_pos: torch.Tensor, token_seq: torch.Tensor, seq_slots: torch.Tensor,
              seq_first_row: Optional[torch.Tensor], xc: torch.Tensor) -> None:
    """xc = silu(causal convolution per channel of the first ``inner`` columns of xz [n, 2 inner]);
    conv_w [inner, taps] (last column: the current token), conv_state [slots, taps - 1, inner]."""
    _cuda(xz, conv_w, conv_b, conv_state, xc, token_pos, token_seq, seq_slots, seq_first_row)
    n, inner = xc.shape
    taps = conv_w.shape[1]
    _need(xz.dtype == xc.dtype and tuple(xz.shape) == (n, 2 * inner), "conv_silu: xz [n, 2 * inner]")
    _need(conv_w.dtype == conv_state.dtype == torch.float32 and conv_w.shape[0] == inner
          and conv_state.dim() == 3 and conv_state.shape[1] >= taps - 1 and conv_state.shape[2] == inner,
          "conv_silu: float32 conv_w [inner, taps], conv_state [slots, taps - 1, inner]")
    _need(conv_state.shape[1] == max(taps - 1, 1), "conv_silu: conv_state holds taps - 1 rows a slot (one at least)")
    _check(_lib().nnis_conv_silu(_ptr(xz), _ptr(conv_w), _ptr(conv_b), _ptr(conv_state), _ptr(token_pos),
                                 _ptr(token_seq), _ptr(seq_slots), _ptr(seq_first_row), _ptr(xc), n, inner, taps,
                                 code_of(xc.dtype), _stream()), "conv_silu")


def selective_scan(xc: torch.Tensor, xz: torch.Tensor, dt_raw: torch.Tensor, bc: torch.Tensor,
                   a_log: torch.Tensor, dskip: torch.Tensor, state: torch.Tensor, conv_state: torch.Tensor,
                   token_pos: torch.Tensor, token_seq: torch.Tensor, seq_slots: torch.Tensor,
                   seq_first_row: Optional[torch.Tensor], seq_count: Optional[torch.Tensor], y: torch.Tensor,
                   taps: int, segments: Optional[torch.Tensor] = None,
                   seq_first_segment: Optional[torch.Tensor] = None, seg_len: int = 0,
                   seg_state: Optional[torch.Tensor] = None, seg_dt: Optional[torch.Tensor] = None) -> None:
    """y = (scan over the step's tokens + D * xc) * silu(z), from and into ``state`` [slots, inner, N];
    moves ``conv_state`` on by the step's inputs.  With ``segments`` (``scan_segments``) a prompt step's
    sequences are cut into runs of ``seg_len`` tokens that are worked side by side; scratch ``seg_state``
    float32 [runs, inner, N] and ``seg_dt`` float32 [runs, inner]."""
    _cuda(xc, xz, dt_raw, bc, a_log, dskip, state, conv_state, y, segments, seq_first_segment, seg_state, seg_dt)
    _seq_tables(token_pos, token_seq, seq_slots, seq_first_row, seq_count)
    n, inner = xc.shape
    N = a_log.shape[1]
    _need(xz.dtype == xc.dtype == y.dtype and tuple(xz.shape) == (n, 2 * inner) and tuple(y.shape) == (n, inner),
          "selective_scan: xc, y [n, inner], xz [n, 2 * inner]")
    _need(dt_raw.dtype == bc.dtype == a_log.dtype == dskip.dtype == state.dtype == torch.float32
          and tuple(dt_raw.shape) == (n, inner) and tuple(bc.shape) == (n, 2 * N) and a_log.shape[0] == inner
          and dskip.numel() == inner and tuple(state.shape[1:]) == (inner, N),
          "selective_scan: float32 dt [n, inner], bc [n, 2 N], A_log [inner, N], D [inner], state")
    _need(N <= 256, f"selective_scan: {N} state values a channel (at most 256)")
    units = seq_first_row.numel() if seq_first_row is not None else n
    n_segments = 0
    if segments is not None:
        n_segments = segments.shape[0]
        _need(seq_first_row is not None and seq_first_segment is not None and seg_len > 0
              and seg_state is not None and seg_state.dtype == torch.float32
              and seg_state.numel() >= n_segments * inner * N and seg_dt is not None
              and seg_dt.dtype == torch.float32 and seg_dt.numel() >= n_segments * inner
              and segments.dtype == seq_first_segment.dtype == torch.int32,
              "selective_scan: runs need a prompt step, their tables and scratch")
    _check(_lib().nnis_selective_scan(_ptr(xc), _ptr(xz), _ptr(dt_raw), _ptr(bc), _ptr(a_log), _ptr(dskip),
                                      _ptr(state), _ptr(conv_state), _ptr(token_pos), _ptr(token_seq),
                                      _ptr(seq_slots), _ptr(seq_first_row), _ptr(seq_count), _ptr(segments),
                                      n_segments, _ptr(seq_first_segment), seg_len, _ptr(seg_state), _ptr(seg_dt),
                                      _ptr(y), units, inner, N, taps, code_of(xc.dtype), _stream()),
           "selective_scan", 3 if segments is not None else 1)


SCAN_SEGMENT = int(os.environ.get("NNIS_SCAN_SEGMENT", "64"))  # tokens of a run of the recurrent mixers; 0: no runs


def scan_segments(counts, seg_len: int):
    """(segments [n, 2] = (sequence, first token of the run), first run of every sequence
    [sequences + 1]) for a prompt step whose sequences bring ``counts`` tokens."""
    return retention_segments(counts, seg_len)


def qkv_prep(a: torch.Tensor, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor],
             freq: Optional[torch.Tensor], token_pos: torch.Tensor, token_seq: torch.Tensor,
             page_table: Optional[torch.Tensor], q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
             v_cache: Optional[torch.Tensor], gate_out: Optional[torch.Tensor], heads: int, kv_heads: int,
             dk: int, dv: int, rot: int, eps: float, pairing: str = "neighbours", head_norm: bool = False,
             q_scale: Optional[torch.Tensor] = None, maps: int = 1, magnitude: float = 1.0) -> None:
    """From float32 rows [q | k | v | gate logits]: norms of q and k, rotation, q packed, k and v into
    the cache, sigmoid of the gate's logits (``gate_out`` [n, heads] or [n, heads * dv]: as many logits a
    row).  ``kv_heads == 0``: the rows hold no keys and values.  Two forms: with ``wq``/``wk`` the
    norms go over the whole projections, before the rotation of neighbouring pairs; with
    ``head_norm``, ``pairing == "half"``, ``q_scale`` (float32 [heads], a multiplier of each head's
    q) or a gate per value, everything is per head: the rotation (either pairing), then optionally
    every head divided by its own root mean square.  ``maps`` > 1: a head of q or k holds that many
    vectors of dk / maps values side by side, each turned by itself over its first ``rot`` values;
    ``magnitude`` multiplies every cosine and sine."""
    _cuda(a, wq, wk, freq, token_pos, token_seq, page_table, q_out, k_cache, v_cache, gate_out, q_scale)
    n = a.shape[0]
    gate_cols = 0 if gate_out is None else gate_out.shape[1]
    _need(gate_cols in (0, heads, heads * dv), "qkv_prep: a gate per head or per value")
    _need(a.dtype == torch.float32 and a.shape[1] == heads * dk + kv_heads * (dk + dv) + gate_cols,
          "qkv_prep: float32 rows [q | k | v | gate]")
    _need(tuple(q_out.shape) == (n, heads * dk), "qkv_prep: q_out [n, heads * dk]")
    for w, size in ((wq, heads * dk), (wk, kv_heads * dk)):
        _need(w is None or (w.dtype == torch.float32 and w.numel() == size), "qkv_prep: float32 norm weights")
    _need(rot == 0 or (freq is not None and freq.dtype == torch.float32 and freq.numel() >= rot // 2),
          "qkv_prep: freq float32 [rot / 2]")
    _need(pairing in ("neighbours", "half"), "qkv_prep: pairing is neighbours or half")
    cols, page_size = 0, 1
    if kv_heads:
        _need(k_cache.dtype == v_cache.dtype == q_out.dtype and tuple(k_cache.shape[1:3]) == tuple(v_cache.shape[1:3])
              and k_cache.shape[1] == kv_heads and k_cache.shape[3] == dk and v_cache.shape[3] == dv,
              "qkv_prep: caches [pages, kv_heads, page, dk] and [.., dv]")
        _need(page_table is not None and page_table.dtype == torch.int32, "qkv_prep: page_table int32")
        cols, page_size = page_table.shape[1], k_cache.shape[2]
    per_head = head_norm or pairing == "half" or q_scale is not None or gate_cols not in (0, heads) \
        or maps != 1 or magnitude != 1.0
    _need(maps >= 1 and dk % maps == 0 and rot <= dk // maps, "qkv_prep: maps vectors of equal size in a head")
    if per_head:
        _need(wq is None and wk is None, "qkv_prep: the per-head form has no norm over the whole projections")
        _need(q_scale is None or (q_scale.dtype == torch.float32 and q_scale.numel() == heads),
              "qkv_prep: q_scale float32 [heads]")
        _check(_lib().nnis_qkv_prep_heads(_ptr(a), _ptr(q_scale), _ptr(freq), _ptr(token_pos), _ptr(token_seq),
                                          _ptr(page_table), cols, _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
                                          _ptr(gate_out), n, heads, kv_heads, dk, dv, rot,
                                          1 if pairing == "half" else 0, 1 if head_norm else 0, gate_cols,
                                          page_size, ctypes.c_float(eps), maps, ctypes.c_float(magnitude),
                                          code_of(q_out.dtype), _stream()),
               "qkv_prep_heads")
        return
    _check(_lib().nnis_qkv_prep(_ptr(a), _ptr(wq), _ptr(wk), _ptr(freq), _ptr(token_pos), _ptr(token_seq),
                                _ptr(page_table), cols, _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _ptr(gate_out),
                                n, heads, kv_heads, dk, dv, rot, 1 if gate_cols else 0, page_size, ctypes.c_float(eps),
                                code_of(q_out.dtype), _stream()), "qkv_prep")


def attention_sink(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, token_pos: torch.Tensor,
                   token_seq: torch.Tensor, page_table: torch.Tensor, sink: Optional[torch.Tensor],
                   gate: Optional[torch.Tensor], out: torch.Tensor, heads: int, kv_heads: int, window: int,
                   chunk: int, scale: float, cap: float, n_splits: int = 1,
                   partial: Optional[torch.Tensor] = None) -> None:
    """Causal attention of packed queries over the paged cache with a soft cap on the scores, a
    chunked and/or windowed mask, a sink per head in the denominator and a gate per (token, head)."""
    _cuda(q, k_cache, v_cache, token_pos, token_seq, page_table, sink, gate, out, partial)
    n = out.shape[0]
    pages, nkv, page_size, dk = k_cache.shape
    dv = v_cache.shape[3]
    _need(nkv == kv_heads and tuple(v_cache.shape[:3]) == (pages, nkv, page_size) and heads % kv_heads == 0,
          "attention_sink: caches [pages, kv_heads, page, dk / dv]")
    _need(q.dtype == k_cache.dtype == v_cache.dtype == out.dtype and tuple(q.shape) == (n, heads * dk)
          and tuple(out.shape) == (n, heads * dv), "attention_sink: q [n, heads * dk], out [n, heads * dv]")
    _need(pages * nkv * page_size < 2 ** 31, "attention_sink: the cache has too many rows")
    _need(sink is None or (sink.dtype == torch.float32 and sink.numel() == heads), "attention_sink: sink [heads]")
    _need(gate is None or (gate.dtype == torch.float32 and gate.numel() >= n * heads), "attention_sink: gate")
    # a gate per (token, head), or, as a matrix [n, heads * dv], per output value
    gate_elems = dv if gate is not None and gate.dim() == 2 and gate.shape[1] == heads * dv and dv > 1 else 0
    if n_splits > 1:
        _need(partial is not None and partial.dtype == torch.float32
              and partial.numel() >= n * heads * n_splits * (dv + 2), "attention_sink: partial scratch")
    _check(_lib().nnis_attention_sink(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(token_pos), _ptr(token_seq),
                                      _ptr(page_table), page_table.shape[1], _ptr(sink), _ptr(gate), _ptr(out),
                                      _ptr(partial), n, heads, kv_heads, dk, dv, page_size, window, chunk,
                                      ctypes.c_float(scale), ctypes.c_float(cap), n_splits, gate_elems,
                                      code_of(out.dtype), _stream()), "attention_sink", 2 if n_splits > 1 else 1)


def attention_sink_mma_takes(dk: int, dv: int, page_size: int) -> bool:
    """Whether the tensor-core prompt form of the sink attention takes these head sizes."""
    return dk == dv and dk in (64, 128) and page_size == 64


def attention_sink_mma(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, tiles: torch.Tensor,
                       seq_first_row: torch.Tensor, seq_start: torch.Tensor, seq_count: torch.Tensor,
                       page_table: torch.Tensor, sink: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                       out: torch.Tensor, heads: int, kv_heads: int, window: int, chunk: int, scale: float,
                       cap: float) -> None:
    """``attention_sink`` for prompt steps in bfloat16 on mma.sync tiles; ``tiles`` int32 [n, 2] =
    (sequence, first query) per 64 queries."""
    _cuda(q, k_cache, v_cache, tiles, seq_first_row, seq_start, seq_count, page_table, sink, gate, out)
    pages, nkv, page_size, d = k_cache.shape
    n = out.shape[0]
    _need(q.dtype == k_cache.dtype == v_cache.dtype == out.dtype == torch.bfloat16, "attention_sink_mma: bfloat16")
    _need(attention_sink_mma_takes(d, v_cache.shape[3], page_size) and nkv == kv_heads,
          "attention_sink_mma: heads of 64 or 128 for keys and values alike, pages of 64")
    _need(tuple(q.shape) == tuple(out.shape) == (n, heads * d), "attention_sink_mma: q, out [n, heads * d]")
    _need(tiles.dtype == torch.int32 and tiles.dim() == 2 and tiles.shape[1] == 2, "attention_sink_mma: tiles [n, 2]")
    _need(sink is None or (sink.dtype == torch.float32 and sink.numel() == heads), "attention_sink_mma: sink")
    _need(gate is None or (gate.dtype == torch.float32 and gate.numel() >= n * heads), "attention_sink_mma: gate")
    gate_elems = d if gate is not None and gate.dim() == 2 and gate.shape[1] == heads * d else 0
    _check(_lib().nnis_attention_sink_mma(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(tiles), tiles.shape[0],
                                          _ptr(seq_first_row), _ptr(seq_start), _ptr(seq_count), _ptr(page_table),
                                          page_table.shape[1], _ptr(sink), _ptr(gate), _ptr(out), heads, kv_heads, d,
                                          page_size, window, chunk, ctypes.c_float(scale), ctypes.c_float(cap),
                                          gate_elems, _stream()), "attention_sink_mma")


def moe_experts_gated(h: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor,
                      weights: torch.Tensor, token_pos: torch.Tensor, act: torch.Tensor,
                      residual: torch.Tensor, top: int) -> None:
    """residual[n] += sum over the chosen experts of W_down[e] (silu(W_gate[e] x) * (W_up[e] x)),
    x = weight * h[n]; w_gu [experts, 2 ff, width], row 2f the gate's and 2f + 1 the up's of feature f."""
    _cuda(h, w_gu, w_down, ids, weights, token_pos, act, residual)
    n, width = h.shape
    experts, ff2, _ = w_gu.shape
    ff = ff2 // 2
    _need(tuple(w_gu.shape) == (experts, 2 * ff, width) and tuple(w_down.shape) == (experts, width, ff)
          and h.dtype == w_gu.dtype == w_down.dtype == act.dtype, "moe_experts_gated: stacked weights of one dtype")
    _need(act.numel() >= n * top * ff, "moe_experts_gated: act scratch [n, top, ff]")
    _need(residual.dtype == torch.float32 and tuple(residual.shape) == (n, width), "moe_experts_gated: residual")
    _check(_lib().nnis_moe_experts_gated(_ptr(h), _ptr(w_gu), _ptr(w_down), _ptr(ids), _ptr(weights),
                                         _ptr(token_pos), _ptr(act), _ptr(residual), n, width, ff, top,
                                         code_of(h.dtype), _stream()), "moe_experts_gated", 2)


def moe_grouped_gated(h: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor,
                      weights: torch.Tensor, perm: torch.Tensor, place: torch.Tensor, tile_expert: torch.Tensor,
                      act: torch.Tensor, y: torch.Tensor, residual: torch.Tensor, top: int, on_output: bool = False,
                      pass_weight: Optional[torch.Tensor] = None) -> None:
    """``moe_experts_gated`` for many tokens in bfloat16: the pairs sorted by expert in runs padded to 64
    rows, two grouped products on mma.sync tiles (the first with the gated activation and the score in
    its epilogue), then the plain sum of each token's experts.  Scratch as ``moe_grouped``."""
    _cuda(h, w_gu, w_down, ids, weights, perm, place, tile_expert, act, y, residual)
    n, width = h.shape
    experts, ff2, _ = w_gu.shape
    ff = ff2 // 2
    tiles = moe_grouped_tiles(n * top, experts)
    _need(h.dtype == w_gu.dtype == w_down.dtype == act.dtype == torch.bfloat16
          and tuple(w_gu.shape) == (experts, 2 * ff, width) and tuple(w_down.shape) == (experts, width, ff),
          "moe_grouped_gated: bfloat16 stacked weights")
    _need(perm.numel() >= tiles * 64 and place.numel() >= n * top and tile_expert.numel() >= tiles
          and act.numel() >= tiles * 64 * ff and y.dtype == torch.float32 and y.numel() >= tiles * 64 * width,
          "moe_grouped_gated: scratch too small")
    _need(residual.dtype == torch.float32 and tuple(residual.shape) == (n, width), "moe_grouped_gated: residual")
    _check(_lib().nnis_moe_grouped_gated(_ptr(h), _ptr(w_gu), _ptr(w_down), _ptr(ids), _ptr(weights), _ptr(perm),
                                         _ptr(place), _ptr(tile_expert), _ptr(act), _ptr(y), _ptr(residual), n, width,
                                         ff, experts, top, 1 if on_output else 0, _ptr(pass_weight), _stream()),
           "moe_grouped_gated", 4)


def moe_grouped_gated_tc(h: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor,
                         weights: torch.Tensor, perm: torch.Tensor, place: torch.Tensor, tile_expert: torch.Tensor,
                         x_sorted: torch.Tensor, up: torch.Tensor, act: torch.Tensor, y: torch.Tensor,
                         residual: torch.Tensor, top: int, on_output: bool = False,
                         pass_weight: Optional[torch.Tensor] = None) -> None:
    """``moe_grouped_gated`` with both products on the tcgen05 kernel: runs padded to tiles of 128 rows
    (``moe_grouped_tc_tiles``); ``up`` float32 [tiles * 128, 2 ff] takes the first product's sums, a row-wise
    kernel applies score and activation.  ``on_output``: the scores weigh the experts' outputs instead, a
    negative id has no expert, and ``pass_weight`` [n] times the token's input is added."""
    _cuda(h, w_gu, w_down, ids, weights, perm, place, tile_expert, x_sorted, up, act, y, residual, pass_weight)
    n, width = h.shape
    experts, ff2, _ = w_gu.shape
    ff = ff2 // 2
    rows = moe_grouped_tc_tiles(n * top, experts) * 128
    _need(h.dtype == w_gu.dtype == w_down.dtype == act.dtype == x_sorted.dtype == torch.bfloat16,
          "moe_grouped_gated_tc: bfloat16")
    _need(tuple(w_gu.shape) == (experts, 2 * ff, width) and tuple(w_down.shape) == (experts, width, ff),
          "moe_grouped_gated_tc: stacked weights")
    _need(moe_grouped_takes(width, ff, experts) and TC_GEMM, "moe_grouped_gated_tc: sizes not taken")
    _need(perm.dtype == place.dtype == tile_expert.dtype == ids.dtype == torch.int32 and perm.numel() >= rows
          and place.numel() >= n * top and tile_expert.numel() >= rows // 128, "moe_grouped_gated_tc: int32 scratch")
    _need(x_sorted.numel() >= rows * width and act.numel() >= rows * ff and y.dtype == up.dtype == torch.float32
          and y.numel() >= rows * width and up.numel() >= rows * 2 * ff, "moe_grouped_gated_tc: scratch")
    _need(residual.dtype == torch.float32 and tuple(residual.shape) == (n, width), "moe_grouped_gated_tc: residual")
    _check(_lib().nnis_moe_grouped_gated_tc(_ptr(h), _ptr(w_gu), _ptr(w_down), _ptr(ids), _ptr(weights), _ptr(perm),
                                            _ptr(place), _ptr(tile_expert), _ptr(x_sorted), _ptr(up), _ptr(act),
                                            _ptr(y), _ptr(residual), n, width, ff, experts, top,
                                            1 if on_output else 0, _ptr(pass_weight),
                                            sm_count(h.device), _ptr(status_word(h.device)), PDL, _stream()),
           "moe_grouped_gated_tc", 6)


GELU_ERF, GELU_TANH, RELU2 = 0, 1, 2


def act_rows(x: torch.Tensor, out: torch.Tensor, kind: int) -> None:
    """out = activation(x), x float32, rounded once to out's dtype; ``GELU_ERF``, ``GELU_TANH`` or ``RELU2``."""
    _cuda(x, out)
    _need(x.dtype == torch.float32 and x.numel() == out.numel(), "act_rows: float32 in, as many values out")
    _check(_lib().nnis_act_rows(_ptr(x), _ptr(out), code_of(out.dtype), ctypes.c_longlong(x.numel()), kind,
                                _stream()), "act_rows")


def depth_mix(hidden: torch.Tensor, history: torch.Tensor, weights: torch.Tensor, terms: int) -> None:
    """history[terms - 1] = hidden; hidden = sum over j < terms of weights[j] * history[j].
    hidden float32 [n, width]; history float32 [at least terms, n, width]; weights float32 [terms]."""
    _cuda(hidden, history, weights)
    _need(hidden.dtype == history.dtype == weights.dtype == torch.float32, "depth_mix: float32")
    _need(history.dim() == 3 and history.shape[0] >= terms and tuple(history.shape[1:]) == tuple(hidden.shape)
          and hidden.is_contiguous() and history.is_contiguous(), "depth_mix: history [terms, n, width]")
    _need(weights.numel() == terms and terms >= 1, "depth_mix: a weight per term")
    _check(_lib().nnis_depth_mix(_ptr(hidden), _ptr(history), _ptr(weights), ctypes.c_longlong(hidden.numel()),
                                 ctypes.c_longlong(hidden.numel()), terms, _stream()), "depth_mix")


def delta_prep(a: torch.Tensor, conv_w: torch.Tensor, tail: torch.Tensor, a_log: torch.Tensor,
               dt_bias: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor, seq_slots: torch.Tensor,
               seq_first_row: Optional[torch.Tensor], seq_count: Optional[torch.Tensor], qkv: torch.Tensor,
               beta_g: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int, unit_eps: float,
               q_scale: float) -> None:
    """What the gated delta rule's recurrence reads, from the projection's float32 rows
    [q | k | v | gate | b | a]: q, k, v through their short causal convolutions (``conv_w``
    [channels, taps], ``tail`` [slots, taps - 1, channels], which is moved on) and silu; q and k heads
    made unit vectors, q times ``q_scale`` (``qkv`` float32 [n, channels]); beta = sigmoid(b) and the
    decay exp(-exp(a_log) softplus(a + dt_bias)) (``beta_g`` float32 [n, 2 heads])."""
    _seq_tables(token_pos, token_seq, seq_slots, seq_first_row, seq_count)
    _cuda(a, conv_w, tail, a_log, dt_bias, qkv, beta_g)
    n = qkv.shape[0]
    channels = 2 * kv_heads * dim + heads * vdim
    taps = conv_w.shape[1]
    _need(a.dtype == torch.float32 and tuple(a.shape) == (n, channels + heads * vdim + 2 * heads),
          "delta_prep: float32 rows [q | k | v | gate | b | a]")
    _need(conv_w.dtype == tail.dtype == torch.float32 and conv_w.shape[0] == channels and conv_w.is_contiguous()
          and tail.dim() == 3 and tuple(tail.shape[1:]) == (max(taps - 1, 1), channels),
          "delta_prep: float32 conv_w [channels, taps], tail [slots, taps - 1, channels]")
    _need(a_log.dtype == dt_bias.dtype == torch.float32 and a_log.numel() == dt_bias.numel() == heads,
          "delta_prep: a_log, dt_bias float32 [heads]")
    _need(qkv.dtype == beta_g.dtype == torch.float32 and qkv.shape[1] == channels
          and tuple(beta_g.shape) == (n, 2 * heads), "delta_prep: qkv [n, channels], beta_g [n, 2 heads] float32")
    units = seq_first_row.numel() if seq_first_row is not None else n
    _check(_lib().nnis_delta_prep(_ptr(a), _ptr(conv_w), _ptr(tail), _ptr(a_log), _ptr(dt_bias), _ptr(token_pos),
                                  _ptr(token_seq), _ptr(seq_slots), _ptr(seq_first_row), _ptr(seq_count), _ptr(qkv),
                                  _ptr(beta_g), n, units, heads, kv_heads, dim, vdim, taps,
                                  ctypes.c_float(unit_eps), ctypes.c_float(q_scale), _stream()),
           "delta_prep", 2 if taps > 1 else 1)


def delta_scan(qkv: torch.Tensor, beta_g: torch.Tensor, state: torch.Tensor, token_pos: torch.Tensor,
               token_seq: torch.Tensor, seq_slots: torch.Tensor, seq_first_row: Optional[torch.Tensor],
               seq_count: Optional[torch.Tensor], o_raw: torch.Tensor, heads: int, kv_heads: int, dim: int,
               vdim: int, segments: Optional[torch.Tensor] = None, seq_first_segment: Optional[torch.Tensor] = None,
               seg_len: int = 0, seg_state: Optional[torch.Tensor] = None, seg_trans: Optional[torch.Tensor] = None,
               q_run: Optional[torch.Tensor] = None) -> None:
    """The gated delta rule over the step's tokens, from and into ``state`` float32
    [slots, heads, dim, vdim]: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  With
    ``segments`` (``scan_segments``) a prompt step's sequences are cut into runs of ``seg_len`` tokens that
    are worked side by side; scratch ``seg_state`` float32 [runs, heads, dim, vdim], ``seg_trans``
    [runs, heads, dim, dim] and ``q_run`` [n, heads, dim]."""
    _seq_tables(token_pos, token_seq, seq_slots, seq_first_row, seq_count)
    _cuda(qkv, beta_g, state, o_raw, segments, seq_first_segment, seg_state, seg_trans, q_run)
    n = qkv.shape[0]
    _need(qkv.dtype == beta_g.dtype == state.dtype == o_raw.dtype == torch.float32, "delta_scan: float32")
    _need(qkv.shape[1] == 2 * kv_heads * dim + heads * vdim and tuple(beta_g.shape) == (n, 2 * heads)
          and tuple(state.shape[1:]) == (heads, dim, vdim) and o_raw.numel() >= n * heads * vdim,
          "delta_scan: qkv [n, channels], beta_g [n, 2 heads], state [slots, heads, dim, vdim]")
    units = seq_first_row.numel() if seq_first_row is not None else n
    n_segments = 0
    if segments is not None:
        n_segments = segments.shape[0]
        _need(seq_first_row is not None and seq_first_segment is not None and seg_len > 0
              and all(t is not None and t.dtype == torch.float32 for t in (seg_state, seg_trans, q_run))
              and seg_state.numel() >= n_segments * heads * dim * vdim
              and seg_trans.numel() >= n_segments * heads * dim * dim and q_run.numel() >= n * heads * dim
              and segments.dtype == seq_first_segment.dtype == torch.int32,
              "delta_scan: runs need a prompt step, their tables and scratch")
    _check(_lib().nnis_delta_scan(_ptr(qkv), _ptr(beta_g), _ptr(state), _ptr(token_pos), _ptr(token_seq),
                                  _ptr(seq_slots), _ptr(seq_first_row), _ptr(seq_count), _ptr(segments), n_segments,
                                  _ptr(seq_first_segment), seg_len, _ptr(seg_state), _ptr(seg_trans), _ptr(q_run),
                                  _ptr(o_raw), units, heads, kv_heads, dim, vdim, _stream()),
           "delta_scan", 3 if segments is not None else 1)


DELTA_SEGMENT = int(os.environ.get("NNIS_DELTA_SEGMENT", "128"))  # tokens of a run of the delta rule; 0: no runs


def delta_finish(o_raw: torch.Tensor, gate_rows: torch.Tensor, gate_off: int, weight: torch.Tensor,
                 token_pos: torch.Tensor, out: torch.Tensor, heads: int, vdim: int, eps: float) -> None:
    """out[n, h] = o[n, h] / rms(o[n, h]) * weight * silu(gate[n, h]); the gate's logits are the
    float32 columns ``gate_off ...`` of ``gate_rows``; ``weight`` float32 [vdim] serves every head."""
    _cuda(o_raw, gate_rows, weight, token_pos, out)
    n = out.shape[0]
    _need(o_raw.dtype == gate_rows.dtype == weight.dtype == torch.float32 and weight.numel() == vdim
          and gate_rows.dim() == 2 and gate_rows.shape[1] >= gate_off + heads * vdim
          and tuple(out.shape) == (n, heads * vdim), "delta_finish: shapes")
    _check(_lib().nnis_delta_finish(_ptr(o_raw), _ptr(gate_rows), gate_rows.shape[1], gate_off, _ptr(weight),
                                    _ptr(token_pos), _ptr(out), n, heads, vdim, ctypes.c_float(eps),
                                    code_of(out.dtype), _stream()), "delta_finish")


# ---------------------------------------------------------------------------
# steps on the stream outside the sub-layers (stream_steps.cu)
# ---------------------------------------------------------------------------
def embed_pair(table: torch.Tensor, pair: Optional[torch.Tensor], tokens: torch.Tensor, token_pos: torch.Tensor,
               token_seq: torch.Tensor, seq_slots: torch.Tensor, seq_count: Optional[torch.Tensor],
               last_token: Optional[torch.Tensor], hidden: torch.Tensor, status: torch.Tensor, scale: float,
               buckets: int, mul_prev: int, mul_cur: int) -> None:
    """hidden[n] = table[token] * scale + pair[(token before * mul_prev + token * mul_cur) mod buckets],
    row ``buckets`` of ``pair`` for a sequence's first token.  The token before a step's first row of a
    sequence is ``last_token[slot]``, which then takes the step's last token of that sequence
    (``seq_count``: tokens per sequence of the step; None: one each).  ``pair`` None: no second table."""
    _cuda(table, pair, tokens, token_pos, token_seq, seq_slots, seq_count, last_token, hidden, status)
    n, width = hidden.shape
    _need(tokens.dtype == torch.int32 and tokens.numel() >= n and token_pos.numel() >= n, "embed_pair: int32 [n]")
    _need(hidden.dtype == torch.float32 and table.shape[1] == width, "embed_pair: hidden float32 [n, width]")
    if pair is not None:
        _need(pair.dtype == table.dtype and tuple(pair.shape) == (buckets + 1, width),
              "embed_pair: pair table [buckets + 1, width] of the table's dtype")
        _need(last_token is not None and last_token.dtype == torch.int32, "embed_pair: last_token int32 [slots]")
    _check(_lib().nnis_embed_pair(_ptr(table), _ptr(pair), code_of(table.dtype), _ptr(tokens), _ptr(token_pos),
                                  _ptr(token_seq), _ptr(seq_slots), _ptr(seq_count), _ptr(last_token), _ptr(hidden),
                                  n, width, table.shape[0], buckets, ctypes.c_longlong(mul_prev),
                                  ctypes.c_longlong(mul_cur), ctypes.c_float(scale), _ptr(status), _stream()),
           "embed_pair")


def rmsnorm_pair(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, eps: float, out1: torch.Tensor,
                 out2: torch.Tensor) -> None:
    """Two RMS norms of the same float32 rows in one pass: out1 = x / rms * w1, out2 = x / rms * w2."""
    _cuda(x, w1, w2, out1, out2)
    n, width = out1.shape
    _need(x.dtype == torch.float32 and tuple(x.shape) == (n, width) and tuple(out2.shape) == (n, width)
          and out1.dtype == out2.dtype, "rmsnorm_pair: x float32 [n, width], two outputs alike")
    _need(w1.dtype == w2.dtype == torch.float32 and w1.numel() == w2.numel() == width,
          "rmsnorm_pair: weights float32 [width]")
    _check(_lib().nnis_rmsnorm_pair(_ptr(x), _ptr(w1), _ptr(w2), _ptr(out1), _ptr(out2), code_of(out1.dtype), n,
                                    width, ctypes.c_float(eps), _stream()), "rmsnorm_pair")


def stream_enter(hidden: torch.Tensor, kept: Optional[torch.Tensor], row: Optional[torch.Tensor]) -> None:
    """hidden += kept (float32, the same shape) + row (float32 [width]); either may be None."""
    _cuda(hidden, kept, row)
    _need(hidden.dtype == torch.float32 and hidden.dim() == 2, "stream_enter: hidden float32 [n, width]")
    _need(kept is None or (kept.dtype == torch.float32 and kept.shape == hidden.shape), "stream_enter: kept")
    _need(row is None or (row.dtype == torch.float32 and row.numel() == hidden.shape[1]), "stream_enter: row")
    _check(_lib().nnis_stream_enter(_ptr(hidden), _ptr(kept), _ptr(row), ctypes.c_longlong(hidden.numel()),
                                    hidden.shape[1], _stream()), "stream_enter")


def scale_rows(x: torch.Tensor, s: float) -> None:
    """x *= s on float32 values."""
    _cuda(x)
    _need(x.dtype == torch.float32, "scale_rows: float32")
    if x.numel():
        _check(_lib().nnis_scale_rows(_ptr(x), ctypes.c_longlong(x.numel()), ctypes.c_float(s), _stream()),
               "scale_rows")


# ---------------------------------------------------------------------------
# differential attention (attention_diff.cu)
# ---------------------------------------------------------------------------
def attention_diff(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, token_pos: torch.Tensor,
                   token_seq: torch.Tensor, page_table: torch.Tensor, gate: Optional[torch.Tensor],
                   out: torch.Tensor, heads: int, kv_heads: int, window: int, scale: float, lam: float,
                   post: float, eps: float, n_splits: int = 1, partial: Optional[torch.Tensor] = None) -> None:
    """Two attention maps a head over the same values: q [n, heads * 2 dk], key rows [k1 | k2] of 2 dk,
    out = rms(a1 - lam * a2) * post * gate over each head's dv values (gate float32 [n, heads * dv])."""
    _cuda(q, k_cache, v_cache, token_pos, token_seq, page_table, gate, out, partial)
    n = out.shape[0]
    pages, nkv, page_size, dk2 = k_cache.shape
    dv = v_cache.shape[3]
    _need(dk2 % 2 == 0 and nkv == kv_heads and tuple(v_cache.shape[:3]) == (pages, nkv, page_size)
          and heads % kv_heads == 0, "attention_diff: caches [pages, kv_heads, page, 2 dk / dv]")
    _need(q.dtype == k_cache.dtype == v_cache.dtype == out.dtype and tuple(q.shape) == (n, heads * dk2)
          and tuple(out.shape) == (n, heads * dv), "attention_diff: q [n, heads * 2 dk], out [n, heads * dv]")
    _need(pages * nkv * page_size < 2 ** 31, "attention_diff: the cache has too many rows")
    _need(gate is None or (gate.dtype == torch.float32 and tuple(gate.shape) == (n, heads * dv)),
          "attention_diff: gate float32 [n, heads * dv]")
    if n_splits > 1:
        _need(partial is not None and partial.dtype == torch.float32
              and partial.numel() >= n * heads * n_splits * (2 * dv + 4), "attention_diff: partial scratch")
    _check(_lib().nnis_attention_diff(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(token_pos), _ptr(token_seq),
                                      _ptr(page_table), page_table.shape[1], _ptr(gate), _ptr(out), _ptr(partial),
                                      n, heads, kv_heads, dk2 // 2, dv, page_size, window, ctypes.c_float(scale),
                                      ctypes.c_float(lam), ctypes.c_float(post), ctypes.c_float(eps), n_splits,
                                      code_of(out.dtype), _stream()), "attention_diff", 2 if n_splits > 1 else 1)


# ---------------------------------------------------------------------------
# experts chosen by corrected scores, group by group (moe.cu)
# ---------------------------------------------------------------------------
def moe_route_choice(h: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor],
                     token_pos: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, pass_weight: torch.Tensor,
                     experts: int, top: int, groups: int = 1, keep: int = 1) -> None:
    """Scores s = softmax over ALL outputs of the router; chosen: the ``top`` largest s + correction among
    the ``keep`` best of ``groups`` equal runs of neighbours; weights = the chosen s, as they are.  Outputs
    from ``experts`` on have no expert: ids -1, their weights summed in ``pass_weight`` [n]."""
    _cuda(h, w_router, correction, token_pos, ids, weights, pass_weight)
    n, width = h.shape
    outputs = w_router.shape[0]
    _need(w_router.dtype == torch.float32 and w_router.shape[1] == width, "moe_route_choice: router float32")
    _need(correction is None or (correction.dtype == torch.float32 and correction.numel() == outputs),
          "moe_route_choice: correction float32 [outputs]")
    _need(ids.dtype == torch.int32 and weights.dtype == pass_weight.dtype == torch.float32
          and ids.numel() >= n * top and weights.numel() >= n * top and pass_weight.numel() >= n,
          "moe_route_choice: ids int32 [n, top], weights float32 [n, top], pass_weight float32 [n]")
    _check(_lib().nnis_moe_route_choice(_ptr(h), _ptr(w_router), _ptr(correction), _ptr(token_pos), _ptr(ids),
                                        _ptr(weights), _ptr(pass_weight), n, width, outputs, experts, top, groups,
                                        keep, code_of(h.dtype), _stream()), "moe_route_choice")


def moe_experts_gated_out(h: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor,
                          weights: torch.Tensor, pass_weight: Optional[torch.Tensor], token_pos: torch.Tensor,
                          act: torch.Tensor, residual: torch.Tensor, top: int) -> None:
    """residual[n] += sum over the chosen experts of weight * W_down[e] (silu(W_gate[e] h) * (W_up[e] h))
    + pass_weight[n] * h[n]; a negative id has no expert."""
    _cuda(h, w_gu, w_down, ids, weights, pass_weight, token_pos, act, residual)
    n, width = h.shape
    experts, ff2, _ = w_gu.shape
    ff = ff2 // 2
    _need(tuple(w_gu.shape) == (experts, 2 * ff, width) and tuple(w_down.shape) == (experts, width, ff)
          and h.dtype == w_gu.dtype == w_down.dtype == act.dtype, "moe_experts_gated_out: stacked weights of one dtype")
    _need(act.numel() >= n * top * ff, "moe_experts_gated_out: act scratch [n, top, ff]")
    _need(residual.dtype == torch.float32 and tuple(residual.shape) == (n, width), "moe_experts_gated_out: residual")
    _check(_lib().nnis_moe_experts_gated_out(_ptr(h), _ptr(w_gu), _ptr(w_down), _ptr(ids), _ptr(weights),
                                             _ptr(pass_weight), _ptr(token_pos), _ptr(act), _ptr(residual), n, width,
                                             ff, top, code_of(h.dtype), _stream()), "moe_experts_gated_out", 2)


DIFF_MMA = 0 if os.environ.get("NNIS_DIFF_MMA", "1") == "0" else 1


def attention_diff_mma_takes(dk: int, dv: int, page_size: int) -> bool:
    """Whether the tensor-core prompt form of differential attention takes maps of ``dk`` values and
    values of ``dv``."""
    return bool(DIFF_MMA) and dk in (32, 64, 128) and dv in (64, 128) and page_size == 64


def attention_diff_mma(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, tiles: torch.Tensor,
                       seq_first_row: torch.Tensor, seq_start: torch.Tensor, seq_count: torch.Tensor,
                       page_table: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, heads: int,
                       kv_heads: int, window: int, scale: float, lam: float, post: float, eps: float) -> None:
    """``attention_diff`` for prompt steps in bfloat16 on mma.sync tiles; ``tiles`` int32 [n, 2] =
    (sequence, first query) per 64 queries."""
    _cuda(q, k_cache, v_cache, tiles, seq_first_row, seq_start, seq_count, page_table, gate, out)
    pages, nkv, page_size, dk2 = k_cache.shape
    dv = v_cache.shape[3]
    n = out.shape[0]
    _need(q.dtype == k_cache.dtype == v_cache.dtype == out.dtype == torch.bfloat16, "attention_diff_mma: bfloat16")
    _need(attention_diff_mma_takes(dk2 // 2, dv, page_size) and nkv == kv_heads and dk2 % 2 == 0,
          "attention_diff_mma: maps of 32, 64 or 128, values of 64 or 128, pages of 64")
    _need(tuple(q.shape) == (n, heads * dk2) and tuple(out.shape) == (n, heads * dv),
          "attention_diff_mma: q [n, heads * 2 dk], out [n, heads * dv]")
    _need(tiles.dtype == torch.int32 and tiles.dim() == 2 and tiles.shape[1] == 2, "attention_diff_mma: tiles [n, 2]")
    _need(gate is None or (gate.dtype == torch.float32 and tuple(gate.shape) == (n, heads * dv)),
          "attention_diff_mma: gate float32 [n, heads * dv]")
    _check(_lib().nnis_attention_diff_mma(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(tiles), tiles.shape[0],
                                          _ptr(seq_first_row), _ptr(seq_start), _ptr(seq_count), _ptr(page_table),
                                          page_table.shape[1], _ptr(gate), _ptr(out), heads, kv_heads, dk2 // 2, dv,
                                          page_size, window, ctypes.c_float(scale), ctypes.c_float(lam),
                                          ctypes.c_float(post), ctypes.c_float(eps), _stream()), "attention_diff_mma")
