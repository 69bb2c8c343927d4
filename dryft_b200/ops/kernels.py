"""Python face of the CUDA kernels: loads the compiled libraries with ``ctypes`` and wraps every
launcher in a function that checks devices, dtypes, shapes and contiguity before the launch.

There is no CPU path and no PyTorch stand-in behind these functions: if the library cannot be
built or loaded, or a tensor is not on a CUDA device, they raise.  (The reference degrades to a
PyTorch path when a Triton kernel fails its self-test, ``engine/dryft_qwen3/model.py:104-119``;
this library fails loudly instead.)

All launches go to PyTorch's current CUDA stream, so they order with PyTorch work and are
captured by ``torch.cuda.graph``.
"""

from __future__ import annotations

import ctypes
import threading
from typing import Dict, Optional, Tuple

import torch

from . import build

_i, _f, _p, _ll, _ull = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_ulonglong

CORE_SOURCES = ("elementwise.cu", "rope_kv.cu", "gemm_f32.cu", "sample.cu", "gemm_small_m.cu", "stream32.cu", "kv_maps.cu", "moe.cu")
UNSUPPORTED = -2


class KernelError(RuntimeError):
    """A launcher refused its arguments or CUDA reported an error at launch."""


_lock = threading.Lock()
_core: Optional[ctypes.CDLL] = None
_variants: Dict[Tuple, ctypes.CDLL] = {}


def _load(path: str) -> ctypes.CDLL:
    try:
        return ctypes.CDLL(path)
    except OSError as e:  # pragma: no cover - depends on the machine
        raise KernelError(f"cannot load compiled kernels {path}: {e}") from e


def core() -> ctypes.CDLL:
    """The size-independent kernels (metadata, embedding, norms, SiLU*mul, RoPE + cache write,
    32-bit matrix product, small-batch bf16 matrix product, token choice)."""
    global _core
    with _lock:
        if _core is None:
            lib = _load(build.build_library("core", CORE_SOURCES))
            lib.dryft_step_meta.argtypes = [_p, _p, _p, _i, _i, _p, _p, _p]
            lib.dryft_step_advance.argtypes = [_p, _p, _p, _i, _p]
            lib.dryft_tokens_from_state.argtypes = [_p, _p, _p, _i, _p]
            lib.dryft_embed.argtypes = [_i, _p, _p, _p, _i, _i, _i, _p, _p]
            lib.dryft_rmsnorm.argtypes = [_i, _p, _p, _p, _p, _p, _p, _i, _i, _f, _p]
            lib.dryft_residual_add.argtypes = [_i, _p, _p, _ll, _p]
            lib.dryft_silu_mul.argtypes = [_i, _p, _p, _i, _i, _p]
            lib.dryft_qk_norm_rope_store.argtypes = [_i, _p, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i,
                                                     _i, _i, _f, _i, _i, _i, _p]
            lib.dryft_rope_table.argtypes = [_i, _p, _p, _p, _i, _i, _p]
            lib.dryft_gemm_nt_f32.argtypes = [_p, _i, _p, _p, _i, _i, _i, _i, _p]
            lib.dryft_argmax_rows.argtypes = [_p, _i, _i, _ll, _p, _p, _p, _p]
            lib.dryft_sample_rows.argtypes = [_p, _i, _i, _ll, _f, _i, _ull, _p, _p, _i, _p, _p, _p, _p]
            lib.dryft_gemm_small_m.argtypes = [_p, _i, _p, _p, _i, _i, _i, _i, _i, _p, _p, _i, _f, _p, _i, _p]
            lib.dryft_row_sumsq.argtypes = [_p, _i, _i, _p, _p, _p, _p]
            lib.dryft_embed_sinusoid.argtypes = [_i, _i, _p, _p, _p, _p, _f, _p, _p, _i, _i, _i, _p, _p]
            lib.dryft_stream_norm_add.argtypes = [_i, _p, _p, _i, _p, _f, _f, _p, _p, _i, _i, _p]
            lib.dryft_stream_norm_rows.argtypes = [_i, _i, _p, _p, _p, _f, _f, _p, _i, _i, _p]
            lib.dryft_kv_maps_store.argtypes = [_i, _p, _i, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p]
            lib.dryft_moe_route.argtypes = [_p, _p, _i, _i, _i, _i, _i, _i, _p, _p, _p]
            lib.dryft_moe_rows.argtypes = [_i, _p, _i, _p, _p, _i, _i, _i, _i, _p, _i, _p, _f, _f, _f, _p]
            lib.dryft_moe_combine.argtypes = [_i, _p, _p, _i, _i, _p, _i, _p]
            lib.dryft_moe_route_rows.argtypes = [_i, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p, _p, _p]
            for name in ("dryft_step_meta", "dryft_step_advance", "dryft_tokens_from_state", "dryft_embed",
                         "dryft_rmsnorm", "dryft_residual_add", "dryft_silu_mul", "dryft_qk_norm_rope_store", "dryft_rope_table",
                         "dryft_gemm_nt_f32", "dryft_argmax_rows", "dryft_sample_rows", "dryft_gemm_small_m", "dryft_row_sumsq",
                         "dryft_embed_sinusoid", "dryft_stream_norm_add", "dryft_stream_norm_rows", "dryft_kv_maps_store",
                         "dryft_moe_route", "dryft_moe_rows", "dryft_moe_combine", "dryft_moe_route_rows"):
                getattr(lib, name).restype = _i
            _core = lib
        return _core


def attention_rows_lib(head_dim: int, group: int, page: int) -> ctypes.CDLL:
    """The row-wise (decode / 32-bit) attention kernel compiled for these sizes."""
    if head_dim <= 0 or head_dim % 16:
        raise KernelError(f"attention kernels take head sizes in steps of 16, got head_dim={head_dim}")
    if head_dim > 256:
        raise KernelError(f"attention kernels take head sizes up to 256, got head_dim={head_dim}")
    if group < 1 or group > 16:
        raise KernelError(f"attention kernels take 1..16 query heads per kv head, got {group}")
    key = ("rows", head_dim, group, page)
    with _lock:
        lib = _variants.get(key)
        if lib is None:
            path = build.build_library("attn_rows", ("attn_rows.cu",),
                                       {"DRYFT_HEAD_DIM": head_dim, "DRYFT_GROUP": group, "DRYFT_PAGE": page})
            lib = _load(path)
            lib.dryft_attn_rows.argtypes = [_i, _p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _i, _i, _i, _f, _i, _p]
            lib.dryft_attn_rows.restype = _i
            if (lib.dryft_attn_rows_head_dim(), lib.dryft_attn_rows_group(), lib.dryft_attn_rows_page()) != (head_dim, group, page):
                raise KernelError(f"{path} was compiled for other sizes")
            _variants[key] = lib
        return lib


def diff_attention_rows_lib(qk_dim: int, v_dim: int, group: int, page: int) -> ctypes.CDLL:
    """The row-wise (decode / 32-bit) differential attention kernel compiled for these sizes."""
    if qk_dim <= 0 or v_dim <= 0 or 2 * qk_dim > 512 or v_dim > 512:
        raise KernelError(f"differential attention takes map sizes up to 256 and value sizes up to 512, got {qk_dim}, {v_dim}")
    if group < 1 or group > 32:
        raise KernelError(f"differential attention takes 1..32 query heads per kv head, got {group}")
    key = ("diff_rows", qk_dim, v_dim, group, page)
    with _lock:
        lib = _variants.get(key)
        if lib is None:
            path = build.build_library("diff_attn_rows", ("diff_attn_rows.cu",),
                                       {"DRYFT_QK_DIM": qk_dim, "DRYFT_V_DIM": v_dim, "DRYFT_GROUP": group, "DRYFT_PAGE": page})
            lib = _load(path)
            lib.dryft_diff_attn_rows.argtypes = [_i, _p, _p, _p, _p, _i, _p, _p, _p, _i, _p, _p, _p, _p, _p, _i, _p, _p, _f, _i, _i, _i,
                                                 _i, _f, _i, _i, _f, _f, _f, _p]
            lib.dryft_diff_attn_rows.restype = _i
            if (lib.dryft_diff_attn_rows_qk_dim(), lib.dryft_diff_attn_rows_v_dim(), lib.dryft_diff_attn_rows_group(),
                    lib.dryft_diff_attn_rows_page()) != (qk_dim, v_dim, group, page):
                raise KernelError(f"{path} was compiled for other sizes")
            _variants[key] = lib
        return lib


def gemm_decode_lib(k: int) -> ctypes.CDLL:
    """The decode matrix product compiled for one inner size ``k`` (a multiple of 256)."""
    if k <= 0 or k % 256:
        raise KernelError(f"the specialised decode product takes inner sizes that are multiples of 256, got {k}")
    key = ("gemm_decode", k)
    with _lock:
        lib = _variants.get(key)
        if lib is None:
            lib = _load(build.build_library("gemm_decode", ("gemm_decode.cu",), {"DRYFT_K": k}))
            lib.dryft_gemm_decode.argtypes = [_p, _i, _p, _p, _i, _i, _i, _i, _p, _p, _i, _f, _p, _i, _i, _p, _p, _p]
            lib.dryft_gemm_decode.restype = _i
            if lib.dryft_gemm_decode_k() != k:
                raise KernelError("the compiled decode product is for another inner size")
            _variants[key] = lib
        return lib


_gemm_stream: Optional[ctypes.CDLL] = None


def gemm_stream_lib() -> ctypes.CDLL:
    """The weight-streaming decode product for up to 64 rows on tcgen05 / TMEM / TMA, work cut evenly over the SMs."""
    global _gemm_stream
    with _lock:
        if _gemm_stream is None:
            lib = _load(build.build_library("gemm_stream", ("gemm_stream.cu",)))
            lib.dryft_gemm_stream.argtypes = [_p, _i, _p, _p, _i, _i, _i, _i, _i, _p, _p, _i, _f, _p, _i, _p, _p, _p, _p]
            lib.dryft_gemm_stream.restype = _i
            lib.dryft_gemm_stream_ss_parts.argtypes = [_i, _i]
            lib.dryft_gemm_stream_ss_parts.restype = _i
            lib.dryft_gemm_stream_workspace_floats.restype = _ll
            _gemm_stream = lib
        return _gemm_stream


_stream_scratch: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}


def gemm_stream_scratch(device: torch.device) -> Tuple[torch.Tensor, torch.Tensor]:
    """(workspace, tickets) of ``gemm_stream`` on this device: float32 slots for the pieces of tiles that two blocks
    share, and zeroed int32 ticket counters (one per tile; every launch leaves them zero).  One set per device
    serves every launch of a stream, because a launch only touches them after the launch before it has ended."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    sc = _stream_scratch.get(idx)
    if sc is None:
        dev = torch.device("cuda", idx)
        with torch.cuda.device(dev):
            n = int(gemm_stream_lib().dryft_gemm_stream_workspace_floats())
        sc = (torch.empty(n, dtype=torch.float32, device=dev), torch.zeros(1 << 16, dtype=torch.int32, device=dev))
        _stream_scratch[idx] = sc
    return sc


def attention_decode_supported(head_dim: int, group: int) -> bool:
    """Whether the one-launch decode attention exists for these sizes (the query heads of a kv head
    form one 16-row tensor-core operand)."""
    return head_dim > 0 and head_dim % 16 == 0 and head_dim <= 256 and 1 <= group <= 16


def attention_decode_lib(head_dim: int, group: int, page: int) -> ctypes.CDLL:
    """The fused decode attention (RoPE + cache write + split attention + combine, bfloat16)."""
    if not attention_decode_supported(head_dim, group):
        raise KernelError(f"fused decode attention does not take head_dim={head_dim} with {group} query heads per kv head")
    key = ("decode", head_dim, group, page)
    with _lock:
        lib = _variants.get(key)
        if lib is None:
            path = build.build_library("attn_decode", ("attn_decode.cu",),
                                       {"DRYFT_HEAD_DIM": head_dim, "DRYFT_GROUP": group, "DRYFT_PAGE": page})
            lib = _load(path)
            lib.dryft_attn_decode.argtypes = [_p, _i, _p, _p, _p, _p, _p, _p, _p, _p, _i, _p, _p, _p, _p, _i, _i, _i, _f, _i,
                                              _i, _f, _i, _i, _i, _i, _i, _p]
            lib.dryft_attn_decode.restype = _i
            _variants[key] = lib
        return lib


def attention_prefill_tc_supported(head_dim: int, group: int, page: int) -> bool:
    """Whether the tcgen05 prefill attention exists for these sizes."""
    return head_dim in (64, 128) and page == 64 and group >= 1


def attention_prefill_tc_lib(head_dim: int, group: int, page: int) -> ctypes.CDLL:
    """The tcgen05 / TMEM / TMA prefill attention compiled for these sizes."""
    if not attention_prefill_tc_supported(head_dim, group, page):
        raise KernelError(f"tcgen05 prefill attention takes head sizes 64 and 128 and 64-token pages, got {head_dim}, {page}")
    key = ("prefill_tc", head_dim, group, page)
    with _lock:
        lib = _variants.get(key)
        if lib is None:
            path = build.build_library("attn_prefill_tc", ("attn_prefill_tc.cu",),
                                       {"DRYFT_HEAD_DIM": head_dim, "DRYFT_GROUP": group, "DRYFT_PAGE": page})
            lib = _load(path)
            lib.dryft_attn_prefill_tc.argtypes = [_p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _f, _i, _p, _p]
            lib.dryft_attn_prefill_tc.restype = _i
            _variants[key] = lib
        return lib


_tickets: Dict[int, torch.Tensor] = {}


def tickets(device: torch.device, n: int) -> torch.Tensor:
    """Zeroed int32 counters the decode attention's blocks draw tickets from; every launch leaves
    them zero again, so one buffer per device serves all layers."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _tickets.get(idx)
    if t is None or t.numel() < n:
        t = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=torch.device("cuda", idx))
        _tickets[idx] = t
    return t


def attention_prefill_lib(head_dim: int, group: int, page: int) -> ctypes.CDLL:
    """The tensor-core prefill attention kernel (bfloat16) compiled for these sizes."""
    if head_dim <= 0 or head_dim % 16 or head_dim > 256:
        raise KernelError(f"prefill attention takes head sizes 16..256 in steps of 16, got head_dim={head_dim}")
    key = ("prefill", head_dim, group, page)
    with _lock:
        lib = _variants.get(key)
        if lib is None:
            path = build.build_library("attn_prefill", ("attn_prefill.cu",),
                                       {"DRYFT_HEAD_DIM": head_dim, "DRYFT_GROUP": group, "DRYFT_PAGE": page})
            lib = _load(path)
            lib.dryft_attn_prefill.argtypes = [_p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _i, _i, _i, _f, _i, _p]
            lib.dryft_attn_prefill.restype = _i
            _variants[key] = lib
        return lib


# ----------------------------------------------------------------------------- argument checks
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> ctypes.c_void_p:
    """The current stream's handle (also inside a graph capture).  A prompt step makes hundreds of launches;
    the raw accessor costs a fraction of a microsecond, the Stream object about fifteen."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> torch.Tensor:
    # the common case first (a prompt step makes a thousand of these checks); what fails it is named below
    try:
        if t.is_cuda and t.is_contiguous() and (dtype is None or t.dtype == dtype) and (
                shape is None or (len(shape) == t.dim() and all(s is None or s == d for s, d in zip(shape, t.shape)))):
            return t
    except AttributeError:
        pass
    if not isinstance(t, torch.Tensor):
        raise KernelError(f"{name}: expected a tensor, got {type(t).__name__}")
    if t.device.type != "cuda":
        raise KernelError(f"{name}: is on {t.device}; dryft_b200 kernels run on a CUDA device only")
    if not t.is_contiguous():
        raise KernelError(f"{name}: must be contiguous (shape {tuple(t.shape)}, strides {t.stride()})")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if shape is not None:
        if len(shape) != t.dim() or any(s is not None and s != d for s, d in zip(shape, t.shape)):
            raise KernelError(f"{name}: expected shape {tuple(shape)}, got {tuple(t.shape)}")
    return t


def _act(t: torch.Tensor, name: str) -> int:
    """1 for bfloat16, 0 for float32; anything else is refused."""
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise KernelError(f"{name}: activations are float32 or bfloat16, got {t.dtype}")


launch_count = 0  # kernels of this library launched (or captured into a graph) so far

_error_flags: Dict[int, torch.Tensor] = {}


def error_flag(device: torch.device) -> torch.Tensor:
    """The device int that kernels with bounded waits raise when a wait runs out."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _error_flags:
        _error_flags[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _error_flags[idx]


_watched: list = []   # (weak reference to a device int32 flag, what a raised flag means)


def watch_flag(flag: torch.Tensor, what: str) -> None:
    """Have ``check_error_flags`` read this device flag too (a part's own error flag, e.g. the embedding's)."""
    import weakref

    _watched.append((weakref.ref(flag), what))


def check_error_flags() -> None:
    """Raise if any kernel gave up a bounded wait, or a part's watched flag was raised, since the last check
    (reads the flags: a sync)."""
    _watched[:] = [(ref, what) for ref, what in _watched if ref() is not None]
    for ref, what in _watched:
        flag = ref()
        if flag is not None and int(flag.item()) != 0:
            flag.zero_()
            raise KernelError(what)
    for idx, flag in _error_flags.items():
        code = int(flag.item())
        if code != 0:
            flag.zero_()
            raise KernelError(f"a kernel on cuda:{idx} gave up waiting for its own copies (bounded wait ran out, "
                              f"place {code}); results since the last check are not valid")


def _ok(rc: int, what: str, n_kernels: int = 1) -> None:
    global launch_count
    if rc == 0:
        launch_count += n_kernels
        return
    if rc == UNSUPPORTED:
        raise KernelError(f"{what}: sizes not supported by this kernel")
    raise KernelError(f"{what}: CUDA error {rc} at launch")


# ----------------------------------------------------------------------------- step metadata
def step_meta(cu_q, seq_slot, seq_len, tok_slot, tok_pos, n_tokens: int, n_seqs: int) -> None:
    for t, n in ((cu_q, "cu_q"), (seq_slot, "seq_slot"), (seq_len, "seq_len"), (tok_slot, "tok_slot"), (tok_pos, "tok_pos")):
        _need(t, n, torch.int32)
    if cu_q.numel() < n_seqs + 1 or seq_slot.numel() < n_seqs or tok_slot.numel() < n_tokens or tok_pos.numel() < n_tokens:
        raise KernelError("step_meta: index arrays shorter than the batch")
    _ok(core().dryft_step_meta(_ptr(cu_q), _ptr(seq_slot), _ptr(seq_len), n_tokens, n_seqs, _ptr(tok_slot), _ptr(tok_pos),
                               _stream()), "step_meta")


def step_advance(cu_q, seq_slot, seq_len, n_seqs: int) -> None:
    for t, n in ((cu_q, "cu_q"), (seq_slot, "seq_slot"), (seq_len, "seq_len")):
        _need(t, n, torch.int32)
    _ok(core().dryft_step_advance(_ptr(cu_q), _ptr(seq_slot), _ptr(seq_len), n_seqs, _stream()), "step_advance")


def tokens_from_state(seq_slot, last_token, tokens, n_seqs: int) -> None:
    for t, n in ((seq_slot, "seq_slot"), (last_token, "last_token"), (tokens, "tokens")):
        _need(t, n, torch.int32)
    _ok(core().dryft_tokens_from_state(_ptr(seq_slot), _ptr(last_token), _ptr(tokens), n_seqs, _stream()), "tokens_from_state")


# ----------------------------------------------------------------------------- elementwise
def embed(tokens, table, out, err=None) -> None:
    _need(tokens, "tokens", torch.int32)
    _need(table, "embedding table")
    n = out.shape[0]
    _need(out, "embedding output", table.dtype, (n, table.shape[1]))
    if tokens.numel() < n:
        raise KernelError("embed: fewer tokens than output rows")
    if err is not None:
        _need(err, "err", torch.int32)
    _ok(core().dryft_embed(_act(table, "embedding table"), _ptr(tokens), _ptr(table), _ptr(out), n, table.shape[1],
                           table.shape[0], _ptr(err), _stream()), "embed")


def rmsnorm(x, weight, eps: float, out, delta=None, rows=None, x_out=None) -> None:
    """``out[r] = norm(x[src] (+ delta[src])) * weight`` with ``src = rows[r]`` if rows is given;
    ``x_out[src]`` receives the summed row when given (may alias ``x``)."""
    hidden = x.shape[-1]
    _need(x, "x")
    _need(weight, "norm weight", torch.float32, (hidden,))
    n_rows = out.shape[0]
    _need(out, "norm output", x.dtype, (n_rows, hidden))
    if delta is not None:
        _need(delta, "delta", x.dtype, tuple(x.shape))
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() < n_rows:
            raise KernelError("rmsnorm: fewer row indices than output rows")
    elif x.shape[0] < n_rows:
        raise KernelError("rmsnorm: input has fewer rows than the output")
    if x_out is not None:
        _need(x_out, "x_out", x.dtype, tuple(x.shape))
    _ok(core().dryft_rmsnorm(_act(x, "x"), _ptr(x), _ptr(delta), _ptr(weight), _ptr(rows), _ptr(x_out), _ptr(out), n_rows,
                             hidden, float(eps), _stream()), f"rmsnorm (width {hidden})")


def residual_add(x, delta) -> None:
    _need(x, "x")
    _need(delta, "delta", x.dtype, tuple(x.shape))
    _ok(core().dryft_residual_add(_act(x, "x"), _ptr(x), _ptr(delta), x.numel(), _stream()), "residual_add")


def silu_mul(gate_up, out) -> None:
    rows, two_i = gate_up.shape
    _need(gate_up, "gate_up")
    if two_i % 2:
        raise KernelError(f"silu_mul: fused gate|up width must be even, got {two_i}")
    _need(out, "silu_mul output", gate_up.dtype, (rows, two_i // 2))
    _ok(core().dryft_silu_mul(_act(gate_up, "gate_up"), _ptr(gate_up), _ptr(out), rows, two_i // 2, _stream()), "silu_mul")


# ----------------------------------------------------------------------------- rope + cache write
def qk_norm_rope_store(qkv, q_norm_w, k_norm_w, inv_freq, tok_slot, tok_pos, q_out, k_pages, v_pages, page_table,
                       n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int, eps: float, write_kv: bool = True,
                       cs_table=None, zero_tail: bool = False) -> None:
    """``cs_table`` (from ``rope_table``; optional) holds the step's cos / sin so that layers share them.
    ``zero_tail``: the last token each sequence brings also zeroes the value rows of its page behind its own
    (what the page's last holder left there), for attention kernels that multiply whole pages."""
    n = qkv.shape[0]
    width = (n_heads + (2 * n_kv_heads if write_kv else 0)) * head_dim
    _need(qkv, "qkv", None, (n, width))
    is_bf16 = _act(qkv, "qkv")
    has_norm = q_norm_w is not None
    if has_norm:
        _need(q_norm_w, "q_norm weight", torch.float32, (head_dim,))
        _need(k_norm_w, "k_norm weight", torch.float32, (head_dim,))
    if rotary_dim:
        _need(inv_freq, "inv_freq", torch.float32, (rotary_dim // 2,))
    _need(tok_slot, "tok_slot", torch.int32)
    _need(tok_pos, "tok_pos", torch.int32)
    if tok_slot.numel() < n or tok_pos.numel() < n:
        raise KernelError("qk_norm_rope_store: token index arrays shorter than the batch")
    _need(q_out, "q_out", qkv.dtype, (n, n_heads, head_dim))
    page_size, max_pages = 0, 0
    if write_kv:
        _need(k_pages, "k_pages", qkv.dtype, (None, n_kv_heads, None, head_dim))
        _need(v_pages, "v_pages", qkv.dtype, tuple(k_pages.shape))
        _need(page_table, "page_table", torch.int32)
        page_size, max_pages = k_pages.shape[2], page_table.shape[1]
    if cs_table is not None:
        _need(cs_table, "cs_table", qkv.dtype, (None, 2, rotary_dim // 2))
        if cs_table.shape[0] < n:
            raise KernelError("qk_norm_rope_store: cos/sin table shorter than the batch")
    _ok(core().dryft_qk_norm_rope_store(is_bf16, _ptr(qkv), width, _ptr(q_norm_w), _ptr(k_norm_w), _ptr(inv_freq),
                                        _ptr(cs_table), _ptr(tok_slot), _ptr(tok_pos), _ptr(q_out), _ptr(k_pages if write_kv else None),
                                        _ptr(v_pages if write_kv else None), _ptr(page_table if write_kv else None),
                                        max_pages, n, n_heads, n_kv_heads, head_dim, rotary_dim, page_size, float(eps),
                                        int(has_norm), int(write_kv), int(zero_tail), _stream()), "qk_norm_rope_store")


def rope_table(tok_pos, inv_freq, n_tokens: int, dtype: torch.dtype) -> torch.Tensor:
    """cos | sin of ``pos * inv_freq`` for every token of a step, rounded to ``dtype``: [n_tokens, 2, R/2]."""
    _need(tok_pos, "tok_pos", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32)
    if tok_pos.numel() < n_tokens:
        raise KernelError("rope_table: tok_pos shorter than the batch")
    half = inv_freq.numel()
    table = torch.empty(n_tokens, 2, half, dtype=dtype, device=tok_pos.device)
    is_bf16 = _act(table, "table")
    _ok(core().dryft_rope_table(is_bf16, _ptr(tok_pos), _ptr(inv_freq), _ptr(table), n_tokens, 2 * half, _stream()), "rope_table")
    return table


# ----------------------------------------------------------------------------- attention
def attn_rows(q, k_pages, v_pages, page_table, tok_slot, tok_pos, out, scale: float, window: Optional[int],
              n_splits: int = 1, part_o=None, part_ml=None) -> None:
    n, n_heads, head_dim = q.shape
    is_bf16 = _act(q, "q")
    _need(q, "q")
    n_kv = k_pages.shape[1]
    page = k_pages.shape[2]
    _need(k_pages, "k_pages", q.dtype, (None, n_kv, page, head_dim))
    _need(v_pages, "v_pages", q.dtype, tuple(k_pages.shape))
    _need(page_table, "page_table", torch.int32)
    _need(tok_slot, "tok_slot", torch.int32)
    _need(tok_pos, "tok_pos", torch.int32)
    if tok_slot.numel() < n or tok_pos.numel() < n:
        raise KernelError("attn_rows: token index arrays shorter than the batch")
    _need(out, "attention output", q.dtype, (n, n_heads * head_dim))
    if n_heads % n_kv:
        raise KernelError(f"attn_rows: {n_heads} query heads are not a multiple of {n_kv} kv heads")
    if n_splits > 1:
        _need(part_o, "part_o", torch.float32)
        _need(part_ml, "part_ml", torch.float32)
        if part_o.numel() < n * n_heads * n_splits * head_dim or part_ml.numel() < n * n_heads * n_splits * 2:
            raise KernelError("attn_rows: partial buffers too small for the split count")
    lib = attention_rows_lib(head_dim, n_heads // n_kv, page)
    _ok(lib.dryft_attn_rows(is_bf16, _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1],
                            _ptr(tok_slot), _ptr(tok_pos), _ptr(out), _ptr(part_o), _ptr(part_ml), n, n_kv, n_splits,
                            float(scale), int(window or 0), _stream()), f"attn_rows (head_dim {head_dim})",
        n_kernels=2 if n_splits > 1 else 1)


def attn_decode(qkv, q_norm_w, k_norm_w, inv_freq, tok_slot, tok_pos, k_pages, v_pages, page_table, out,
                n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int, eps: float, scale: float,
                window: Optional[int], n_splits: int, part_o=None, part_ml=None, write_kv: bool = True, pdl: bool = False,
                shape: int = -1, cluster: bool = True) -> None:
    """One launch for a decode step's attention (bfloat16): per-head q/k norm + RoPE of each row's new
    token, its K/V written into the cache, attention of its query heads over the cache, splits combined.
    ``shape``: warps per block, 0 / 1 / 2 for 8 / 4 / 2; -1 lets the launcher take the widest whose grid is
    resident at once.  ``cluster``: with 2..8 splits the splits of a (row, kv head) run as one thread-block
    cluster and are combined through distributed shared memory (no partial buffers needed); with more
    splits, or ``cluster=False``, they meet in ``part_o`` / ``part_ml`` and the last block to finish combines."""
    n = qkv.shape[0]
    width = (n_heads + (2 * n_kv_heads if write_kv else 0)) * head_dim
    _need(qkv, "qkv", torch.bfloat16, (n, width))
    has_norm = q_norm_w is not None
    if has_norm:
        _need(q_norm_w, "q_norm weight", torch.float32, (head_dim,))
        _need(k_norm_w, "k_norm weight", torch.float32, (head_dim,))
    if rotary_dim:
        _need(inv_freq, "inv_freq", torch.float32, (rotary_dim // 2,))
    page = k_pages.shape[2]
    _need(k_pages, "k_pages", torch.bfloat16, (None, n_kv_heads, page, head_dim))
    _need(v_pages, "v_pages", torch.bfloat16, tuple(k_pages.shape))
    for t, nm in ((page_table, "page_table"), (tok_slot, "tok_slot"), (tok_pos, "tok_pos")):
        _need(t, nm, torch.int32)
    if tok_slot.numel() < n or tok_pos.numel() < n:
        raise KernelError("attn_decode: token index arrays shorter than the batch")
    _need(out, "attention output", torch.bfloat16, (n, n_heads * head_dim))
    if n_heads % n_kv_heads:
        raise KernelError(f"attn_decode: {n_heads} query heads are not a multiple of {n_kv_heads} kv heads")
    tk = None
    use_cluster = bool(cluster) and 2 <= n_splits <= 8
    if n_splits > 1 and not use_cluster:
        _need(part_o, "part_o", torch.float32)
        _need(part_ml, "part_ml", torch.float32)
        if part_o.numel() < n * n_heads * n_splits * head_dim or part_ml.numel() < n * n_heads * n_splits * 2:
            raise KernelError("attn_decode: partial buffers too small for the split count")
        tk = tickets(qkv.device, n * n_kv_heads)
    lib = attention_decode_lib(head_dim, n_heads // n_kv_heads, page)
    _ok(lib.dryft_attn_decode(_ptr(qkv), width, _ptr(q_norm_w), _ptr(k_norm_w), _ptr(inv_freq), _ptr(tok_slot), _ptr(tok_pos),
                              _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1], _ptr(out), _ptr(part_o),
                              _ptr(part_ml), _ptr(tk), n, n_kv_heads, n_splits, float(scale), int(window or 0),
                              int(rotary_dim), float(eps), int(has_norm), int(write_kv), int(pdl), int(shape), int(use_cluster), _stream()),
        f"attn_decode (head_dim {head_dim})")


def attn_prefill(q, k_pages, v_pages, page_table, tile_tok0, tile_rows, tok_slot, tok_pos, out, n_tiles: int,
                 scale: float, window: Optional[int]) -> None:
    """Causal grouped-query attention of packed prompts over the paged cache (bfloat16, tensor cores).
    Tile ``t`` covers the ``tile_rows[t]`` query tokens from packed index ``tile_tok0[t]`` on, all of one
    sequence; their slot and positions are read from ``tok_slot`` / ``tok_pos``."""
    n, n_heads, head_dim = q.shape
    _need(q, "q", torch.bfloat16)
    n_kv = k_pages.shape[1]
    page = k_pages.shape[2]
    _need(k_pages, "k_pages", torch.bfloat16, (None, n_kv, page, head_dim))
    _need(v_pages, "v_pages", torch.bfloat16, tuple(k_pages.shape))
    for t, nm in ((page_table, "page_table"), (tile_tok0, "tile_tok0"), (tile_rows, "tile_rows"),
                  (tok_slot, "tok_slot"), (tok_pos, "tok_pos")):
        _need(t, nm, torch.int32)
    if tile_tok0.numel() < n_tiles or tile_rows.numel() < n_tiles:
        raise KernelError("attn_prefill: tile arrays shorter than the tile count")
    _need(out, "attention output", torch.bfloat16, (n, n_heads * head_dim))
    if n_heads % n_kv:
        raise KernelError(f"attn_prefill: {n_heads} query heads are not a multiple of {n_kv} kv heads")
    lib = attention_prefill_lib(head_dim, n_heads // n_kv, page)
    _ok(lib.dryft_attn_prefill(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1],
                               _ptr(tile_tok0), _ptr(tile_rows), _ptr(tok_slot), _ptr(tok_pos), _ptr(out), n_tiles,
                               n_heads, n_kv, float(scale), int(window or 0), _stream()),
        f"attn_prefill (head_dim {head_dim})")


def attn_prefill_tc(q, k_pages, v_pages, page_table, tile_tok0, tile_rows, tok_slot, tok_pos, out, n_tiles: int,
                    scale: float, window: Optional[int]) -> None:
    """``attn_prefill`` on the 5th-generation tensor cores (tcgen05.mma, tensor memory, TMA); tiles of up
    to 128 query tokens; head sizes 64 and 128."""
    n, n_heads, head_dim = q.shape
    _need(q, "q", torch.bfloat16)
    n_kv = k_pages.shape[1]
    page = k_pages.shape[2]
    _need(k_pages, "k_pages", torch.bfloat16, (None, n_kv, page, head_dim))
    _need(v_pages, "v_pages", torch.bfloat16, tuple(k_pages.shape))
    for t, nm in ((page_table, "page_table"), (tile_tok0, "tile_tok0"), (tile_rows, "tile_rows"),
                  (tok_slot, "tok_slot"), (tok_pos, "tok_pos")):
        _need(t, nm, torch.int32)
    if tile_tok0.numel() < n_tiles or tile_rows.numel() < n_tiles:
        raise KernelError("attn_prefill_tc: tile arrays shorter than the tile count")
    _need(out, "attention output", torch.bfloat16, (n, n_heads * head_dim))
    if n_heads % n_kv:
        raise KernelError(f"attn_prefill_tc: {n_heads} query heads are not a multiple of {n_kv} kv heads")
    lib = attention_prefill_tc_lib(head_dim, n_heads // n_kv, page)
    _ok(lib.dryft_attn_prefill_tc(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1],
                                  _ptr(tile_tok0), _ptr(tile_rows), _ptr(tok_slot), _ptr(tok_pos), _ptr(out), n_tiles, n,
                                  k_pages.shape[0], n_heads, n_kv, float(scale), int(window or 0),
                                  _ptr(error_flag(q.device)), _stream()),
        f"attn_prefill_tc (head_dim {head_dim})")


# ----------------------------------------------------------------------------- 32-bit residual stream
def embed_sinusoid(tokens, tok_pos, table, freq, scale: float, x32, h=None, err=None) -> None:
    """``x32[n] = table[tokens[n]] * scale + s(tok_pos[n])`` with ``s[2i] = sin(pos * freq[i])``, ``s[2i+1] = cos`` of the
    same angle; ``h`` (optional, bfloat16 or float32) receives the row rounded to its type."""
    n, width = x32.shape
    _need(tokens, "tokens", torch.int32)
    _need(tok_pos, "tok_pos", torch.int32)
    _need(table, "embedding table", None, (None, width))
    _need(freq, "freq", torch.float32, ((width + 1) // 2,))
    _need(x32, "stream", torch.float32)
    if tokens.numel() < n or tok_pos.numel() < n:
        raise KernelError("embed_sinusoid: fewer tokens than rows")
    if h is not None:
        _need(h, "h", None, (n, width))
    if err is not None:
        _need(err, "err", torch.int32)
    _ok(core().dryft_embed_sinusoid(_act(table, "embedding table"), _act(h, "h") if h is not None else 0, _ptr(tokens), _ptr(tok_pos),
                                    _ptr(table), _ptr(freq), float(scale), _ptr(x32), _ptr(h), n, width, table.shape[0], _ptr(err),
                                    _stream()), "embed_sinusoid")


def stream_norm_add(y, weight, offset: float, eps: float, x32, h=None, wts=None, top: int = 0) -> None:
    """``x32[n] += y[n] / sqrt(mean(y[n]^2) + eps) * (offset + weight)`` in 32-bit; ``h`` (optional, of ``y``'s type) receives
    the new row rounded.  With ``wts`` ``[n, top]`` float32, ``y`` is ``[n * top, width]`` and row ``n`` is the weighted sum
    ``sum_k wts[n, k] * y[n * top + k]`` (formed in 32-bit)."""
    n, width = x32.shape
    _need(x32, "stream", torch.float32)
    _need(weight, "norm weight", torch.float32, (width,))
    if wts is not None:
        if top <= 0:
            raise KernelError("stream_norm_add: wts needs top > 0")
        _need(wts, "wts", torch.float32, (n, top))
        _need(y, "y", None, (n * top, width))
    else:
        top = 0
        _need(y, "y", None, (n, width))
    if h is not None:
        _need(h, "h", y.dtype, (n, width))
    _ok(core().dryft_stream_norm_add(_act(y, "y"), _ptr(y), _ptr(wts), int(top), _ptr(weight), float(offset), float(eps), _ptr(x32),
                                     _ptr(h), n, width, _stream()), f"stream_norm_add (width {width})")


def stream_norm_rows(x, weight, offset: float, eps: float, out, rows=None) -> None:
    """``out[r] = norm(x[src]) * (offset + weight)`` with ``src = rows[r]`` if rows is given; ``x`` and ``out`` are float32 or
    bfloat16 independently."""
    width = x.shape[-1]
    _need(x, "x")
    _need(weight, "norm weight", torch.float32, (width,))
    n = out.shape[0]
    _need(out, "norm output", None, (n, width))
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() < n:
            raise KernelError("stream_norm_rows: fewer row indices than output rows")
    elif x.shape[0] < n:
        raise KernelError("stream_norm_rows: input has fewer rows than the output")
    _ok(core().dryft_stream_norm_rows(_act(x, "x"), _act(out, "out"), _ptr(x), _ptr(rows), _ptr(weight), float(offset), float(eps),
                                      _ptr(out), n, width, _stream()), f"stream_norm_rows (width {width})")


# ----------------------------------------------------------------------------- differential attention
def kv_maps_store(proj, q_norm_w, k_norm_w, tok_slot, tok_pos, q_out, k_pages, v_pages, page_table, n_heads: int,
                  n_kv_heads: int, maps: int, dim: int, v_dim: int, eps: float, write_kv: bool = True) -> None:
    """Rows of ``proj`` are ``[q: heads x maps x dim | k: kv_heads x maps x dim | v: kv_heads x v_dim | ...]`` (k and v absent
    without ``write_kv``).  Every (head, map) vector of q and k gets its RMS norm (weights ``[dim]``, optional); q goes to
    ``q_out [n, heads, maps*dim]``, k and v into the paged cache at each token's (slot, position)."""
    n = proj.shape[0]
    need_w = n_heads * maps * dim + ((n_kv_heads * maps * dim + n_kv_heads * v_dim) if write_kv else 0)
    _need(proj, "proj")
    if proj.dim() != 2 or proj.shape[1] < need_w:
        raise KernelError(f"kv_maps_store: projection rows have {tuple(proj.shape)}, need at least {need_w} columns")
    is_bf16 = _act(proj, "proj")
    for w_, nm in ((q_norm_w, "q norm weight"), (k_norm_w, "k norm weight")):
        if w_ is not None:
            _need(w_, nm, torch.float32, (dim,))
    _need(tok_slot, "tok_slot", torch.int32)
    _need(tok_pos, "tok_pos", torch.int32)
    if tok_slot.numel() < n or tok_pos.numel() < n:
        raise KernelError("kv_maps_store: token index arrays shorter than the batch")
    _need(q_out, "q_out", proj.dtype, (n, n_heads, maps * dim))
    page_size = max_pages = 0
    if write_kv:
        _need(k_pages, "k_pages", proj.dtype, (None, n_kv_heads, None, maps * dim))
        _need(v_pages, "v_pages", proj.dtype, (k_pages.shape[0], n_kv_heads, k_pages.shape[2], v_dim))
        _need(page_table, "page_table", torch.int32)
        page_size, max_pages = k_pages.shape[2], page_table.shape[1]
    _ok(core().dryft_kv_maps_store(is_bf16, _ptr(proj), proj.shape[1], _ptr(q_norm_w), _ptr(k_norm_w), _ptr(tok_slot), _ptr(tok_pos),
                                   _ptr(q_out), _ptr(k_pages if write_kv else None), _ptr(v_pages if write_kv else None),
                                   _ptr(page_table if write_kv else None), max_pages, n, n_heads, n_kv_heads, maps, dim, v_dim,
                                   page_size, float(eps), int(write_kv), _stream()), "kv_maps_store")


def diff_attn_rows(q, k_pages, v_pages, page_table, tok_slot, tok_pos, out, scale: float, lam: float, sub_eps: float,
                   out_scale: float, window: Optional[int] = None, chunk: Optional[int] = None, gate=None, gate_col: int = 0,
                   n_splits: int = 1, part_o=None, part_ml=None, proj=None, n_heads: int = 0, q_norm_w=None, k_norm_w=None,
                   qk_eps: float = 0.0, write_kv: bool = False) -> None:
    """Differential attention of independent rows: ``q [n, heads, 2*dim]`` (normalised), keys ``[pages, kv, page, 2*dim]``,
    values ``[pages, kv, page, v_dim]``; ``out [n, heads*v_dim] = gate * out_scale * unit_rms(a1 - lam * a2)``.  ``gate``: a
    2-D tensor whose columns ``gate_col .. gate_col + heads - 1`` hold one logit per head (sigmoid is applied).

    With ``proj`` instead of ``q`` (a step whose rows are each their sequence's one new token): rows of ``proj`` are
    ``[q | k | v | ...]`` as ``kv_maps_store`` takes them, the per-map norm of the ``n_heads`` queries happens inside, and
    with ``write_kv`` so do the norm and the cache write of each row's new key and value -- one launch for all of it."""
    if proj is not None:
        if q is not None or n_heads <= 0:
            raise KernelError("diff_attn_rows: give either q or (proj, n_heads)")
        n, kw = proj.shape[0], k_pages.shape[3]
        _need(proj, "proj", k_pages.dtype)
        is_bf16 = _act(proj, "proj")
        need_w = n_heads * kw + ((k_pages.shape[1] * kw + k_pages.shape[1] * v_pages.shape[3]) if write_kv else 0)
        if proj.dim() != 2 or proj.shape[1] < need_w:
            raise KernelError(f"diff_attn_rows: projection rows have {tuple(proj.shape)}, need at least {need_w} columns")
        for w_, nm in ((q_norm_w, "q norm weight"), (k_norm_w, "k norm weight")):
            if w_ is not None:
                _need(w_, nm, torch.float32, (kw // 2,))
        q_dtype = proj.dtype
    else:
        n, n_heads, kw = q.shape
        is_bf16 = _act(q, "q")
        _need(q, "q")
        q_dtype = q.dtype
    n_kv, page, v_dim = k_pages.shape[1], k_pages.shape[2], v_pages.shape[3]
    _need(k_pages, "k_pages", q_dtype, (None, n_kv, page, kw))
    _need(v_pages, "v_pages", q_dtype, (k_pages.shape[0], n_kv, page, v_dim))
    for t, nm in ((page_table, "page_table"), (tok_slot, "tok_slot"), (tok_pos, "tok_pos")):
        _need(t, nm, torch.int32)
    if tok_slot.numel() < n or tok_pos.numel() < n:
        raise KernelError("diff_attn_rows: token index arrays shorter than the batch")
    _need(out, "attention output", q_dtype, (n, n_heads * v_dim))
    if n_heads % n_kv or kw % 2:
        raise KernelError(f"diff_attn_rows: {n_heads} query heads / {n_kv} kv heads / key rows of {kw}")
    gate_ptr, gate_stride = None, 0
    if gate is not None:
        _need(gate, "gate", q_dtype)
        if gate.dim() != 2 or gate.shape[0] < n or gate.shape[1] < gate_col + n_heads:
            raise KernelError("diff_attn_rows: gate columns outside the gate tensor")
        gate_ptr, gate_stride = ctypes.c_void_p(gate.data_ptr() + gate_col * gate.element_size()), gate.shape[1]
    if n_splits > 1:
        _need(part_o, "part_o", torch.float32)
        _need(part_ml, "part_ml", torch.float32)
        if part_o.numel() < n * n_heads * 2 * n_splits * v_dim or part_ml.numel() < n * n_heads * 2 * n_splits * 2:
            raise KernelError("diff_attn_rows: partial buffers too small for the split count")
    tk = tickets(out.device, n * n_kv) if n_splits > 1 else None   # zeroed counters; every launch leaves them zero
    fuse = 0 if proj is None else (2 if write_kv else 1)
    lib = diff_attention_rows_lib(kw // 2, v_dim, n_heads // n_kv, page)
    _ok(lib.dryft_diff_attn_rows(is_bf16, _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1], _ptr(tok_slot),
                                 _ptr(tok_pos), gate_ptr, gate_stride, _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(tk), _ptr(proj),
                                 proj.shape[1] if proj is not None else 0, _ptr(q_norm_w), _ptr(k_norm_w), float(qk_eps), fuse, n, n_kv,
                                 n_splits, float(scale), int(window or 0), int(chunk or 0), float(lam), float(sub_eps),
                                 float(out_scale), _stream()), f"diff_attn_rows (dims {kw // 2}, {v_dim})")


# ----------------------------------------------------------------------------- mixture of experts
def _route_flags(renorm: bool, score: str) -> int:
    if score not in ("softmax", "sigmoid"):
        raise KernelError(f"moe_route: scores are 'softmax' or 'sigmoid', got {score!r}")
    return int(bool(renorm)) | (2 if score == "sigmoid" else 0)


def moe_route(logits, n_groups: int, keep: int, top: int, idx_out, w_out, renorm: bool = False, bias=None, score: str = "softmax") -> None:
    """The router's choice per token from 32-bit ``logits [n, experts]`` (plus ``bias [experts]``, if given): ``idx_out [n, top]``
    int32, ``w_out [n, top]`` float32.  ``renorm``: the chosen scores divided by their sum (a softmax over the chosen logits).
    ``score="sigmoid"``: an expert's score is the sigmoid of its own logit instead of the softmax over all of them."""
    n, e = logits.shape
    _need(logits, "router logits", torch.float32)
    if bias is not None:
        _need(bias, "router bias", torch.float32, (e,))
    _need(idx_out, "idx_out", torch.int32, (n, top))
    _need(w_out, "w_out", torch.float32, (n, top))
    _ok(core().dryft_moe_route(_ptr(logits), _ptr(bias), n, e, int(n_groups), int(keep), int(top), _route_flags(renorm, score), _ptr(idx_out), _ptr(w_out),
                               _stream()), f"moe_route ({e} experts, {n_groups} groups, keep {keep}, top {top})")


def moe_route_rows_supported(hidden: int, experts: int, groups: int, itemsize: int) -> bool:
    """Whether the one-launch router (product and choice) takes these sizes: its row and scores fit 48 KB of shared memory."""
    return 4 * (2 * experts + groups) + (itemsize * hidden + 15) // 16 * 16 <= 48 * 1024


def moe_route_rows(h, w_router, n_groups: int, keep: int, top: int, idx_out, w_out, renorm: bool = False, bias=None,
                   score: str = "softmax") -> None:
    """``moe_route`` of ``logits = h @ w_router.T`` (32-bit sums) in one launch, for few tokens: one block per token."""
    n, k = h.shape
    e = w_router.shape[0]
    _need(h, "h")
    _need(w_router, "router weight", h.dtype, (e, k))
    _need(idx_out, "idx_out", torch.int32, (n, top))
    _need(w_out, "w_out", torch.float32, (n, top))
    if bias is not None:
        _need(bias, "router bias", torch.float32, (e,))
    _ok(core().dryft_moe_route_rows(_act(h, "h"), _ptr(h), _ptr(w_router), _ptr(bias), n, k, e, int(n_groups), int(keep), int(top), _route_flags(renorm, score),
                                    _ptr(idx_out), _ptr(w_out), _stream()), f"moe_route_rows ({e} experts over {k})")


def moe_rows(a, w, idx, out, mode: str, in_w=None, limit: Optional[float] = None, alpha: float = 1.0, up_offset: float = 0.0) -> None:
    """Experts evaluated assignment by assignment.  ``idx [n, top]`` int32 names each assignment's expert.
    ``mode="gate_up_clamp"``: as ``gate_up`` with the assignment's weight ``s = in_w[n, k]`` on the expert's input and a clamped
    activation: ``g = min(s * gate, limit)``, ``u = clamp(s * up, -limit, limit)``, ``out = g * sigmoid(alpha * g) * (u + up_offset)``;
    ``mode="gate_up"``: ``a [n, K]`` token rows, ``w [E, 2F, K]``, ``out [n*top, F] = silu(gate) * up``;
    ``mode="down"``: ``a [n*top, F]``, ``w [E, C, F]``, ``out [n*top, C]``;
    ``mode="up_relu2"`` (experts without a gate): ``a [n, K]``, ``w [E, F, K]``, ``out [n*top, F] = max(up, 0)^2``."""
    n_assign = idx.numel()
    _need(idx, "idx", torch.int32)
    is_bf16 = _act(a, "a")
    _need(a, "a")
    _need(w, "w", a.dtype)
    e, r, k = w.shape
    if mode in ("gate_up", "gate_up_clamp"):
        top = idx.shape[1]
        n_out, code, a_div = r // 2, (0 if mode == "gate_up" else 3), top
        if mode == "gate_up_clamp":
            _need(in_w, "in_w", torch.float32, tuple(idx.shape))
        if a.shape != (idx.shape[0], k) or r % 2:
            raise KernelError(f"moe_rows: activations {tuple(a.shape)} against weights {tuple(w.shape)}")
    elif mode == "up_relu2":
        n_out, code, a_div = r, 2, idx.shape[1]
        if a.shape != (idx.shape[0], k):
            raise KernelError(f"moe_rows: activations {tuple(a.shape)} against weights {tuple(w.shape)}")
    elif mode == "down":
        n_out, code, a_div = r, 1, 1
        if a.shape != (n_assign, k):
            raise KernelError(f"moe_rows: activations {tuple(a.shape)} against weights {tuple(w.shape)}")
    else:
        raise KernelError(f"moe_rows: unknown mode {mode!r}")
    _need(out, "out", a.dtype, (n_assign, n_out))
    _ok(core().dryft_moe_rows(is_bf16, _ptr(a), a_div, _ptr(w), _ptr(idx), e, k, n_out, code, _ptr(out), n_assign,
                              _ptr(in_w if code == 3 else None), float("inf") if limit is None else float(limit), float(alpha),
                              float(up_offset), _stream()),
        f"moe_rows ({mode}, K={k}, out={n_out})")


def moe_combine(y, wts, out) -> None:
    """``out[n] = sum_k wts[n, k] * y[n * top + k]``."""
    n, top = wts.shape
    _need(wts, "wts", torch.float32)
    _need(y, "y", None, (n * top, out.shape[1]))
    _need(out, "out", y.dtype, (n, y.shape[1]))
    _ok(core().dryft_moe_combine(_act(y, "y"), _ptr(y), _ptr(wts), top, y.shape[1], _ptr(out), n, _stream()), "moe_combine")


def diff_attention_prefill_supported(qk_dim: int, v_dim: int, group: int, page: int) -> bool:
    """Whether the tensor-core differential prompt attention exists for these sizes (k16 steps over a map, n8 pairs over
    the values, 64-token pages)."""
    return (qk_dim > 0 and qk_dim % 16 == 0 and qk_dim <= 128 and v_dim > 0 and v_dim % 16 == 0 and v_dim <= 256
            and page == 64 and group >= 1 and 2 * ((64 + 128) * (2 * qk_dim + 8) + 128 * (v_dim + 8)) <= 227 * 1024)


def diff_attention_prefill_lib(qk_dim: int, v_dim: int, group: int, page: int) -> ctypes.CDLL:
    if not diff_attention_prefill_supported(qk_dim, v_dim, group, page):
        raise KernelError(f"differential prompt attention takes map and value sizes in steps of 16 and 64-token pages, got "
                          f"{qk_dim}, {v_dim}, {page}")
    key = ("diff_prefill", qk_dim, v_dim, group, page)
    with _lock:
        lib = _variants.get(key)
        if lib is None:
            path = build.build_library("diff_attn_prefill", ("diff_attn_prefill.cu",),
                                       {"DRYFT_QK_DIM": qk_dim, "DRYFT_V_DIM": v_dim, "DRYFT_GROUP": group, "DRYFT_PAGE": page})
            lib = _load(path)
            lib.dryft_diff_attn_prefill.argtypes = [_p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _i, _p, _i, _i, _i, _f, _i, _i, _f, _f, _f, _p]
            lib.dryft_diff_attn_prefill.restype = _i
            if (lib.dryft_diff_attn_prefill_qk_dim(), lib.dryft_diff_attn_prefill_v_dim()) != (qk_dim, v_dim):
                raise KernelError(f"{path} was compiled for other sizes")
            _variants[key] = lib
        return lib


def diff_attn_prefill(q, k_pages, v_pages, page_table, tile_tok0, tile_rows, tok_slot, tok_pos, out, n_tiles: int, scale: float,
                      lam: float, sub_eps: float, out_scale: float, window: Optional[int] = None, chunk: Optional[int] = None,
                      gate=None, gate_col: int = 0) -> None:
    """``diff_attn_rows``'s result for packed prompts (bfloat16, tensor cores).  Tile ``t`` covers the ``tile_rows[t]`` query
    tokens from packed index ``tile_tok0[t]`` on, all of one sequence."""
    n, n_heads, kw = q.shape
    _need(q, "q", torch.bfloat16)
    n_kv, page, v_dim = k_pages.shape[1], k_pages.shape[2], v_pages.shape[3]
    _need(k_pages, "k_pages", torch.bfloat16, (None, n_kv, page, kw))
    _need(v_pages, "v_pages", torch.bfloat16, (k_pages.shape[0], n_kv, page, v_dim))
    for t, nm in ((page_table, "page_table"), (tile_tok0, "tile_tok0"), (tile_rows, "tile_rows"), (tok_slot, "tok_slot"),
                  (tok_pos, "tok_pos")):
        _need(t, nm, torch.int32)
    if tile_tok0.numel() < n_tiles or tile_rows.numel() < n_tiles:
        raise KernelError("diff_attn_prefill: tile arrays shorter than the tile count")
    _need(out, "attention output", torch.bfloat16, (n, n_heads * v_dim))
    if n_heads % n_kv or kw % 2:
        raise KernelError(f"diff_attn_prefill: {n_heads} query heads / {n_kv} kv heads / key rows of {kw}")
    gate_ptr, gate_stride = None, 0
    if gate is not None:
        _need(gate, "gate", torch.bfloat16)
        if gate.dim() != 2 or gate.shape[0] < n or gate.shape[1] < gate_col + n_heads:
            raise KernelError("diff_attn_prefill: gate columns outside the gate tensor")
        gate_ptr, gate_stride = ctypes.c_void_p(gate.data_ptr() + gate_col * gate.element_size()), gate.shape[1]
    lib = diff_attention_prefill_lib(kw // 2, v_dim, n_heads // n_kv, page)
    _ok(lib.dryft_diff_attn_prefill(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1], _ptr(tile_tok0),
                                    _ptr(tile_rows), _ptr(tok_slot), _ptr(tok_pos), gate_ptr, gate_stride, _ptr(out), n_tiles,
                                    n_heads, n_kv, float(scale), int(window or 0), int(chunk or 0), float(lam), float(sub_eps),
                                    float(out_scale), _stream()), f"diff_attn_prefill (dims {kw // 2}, {v_dim})")


_moe_grouped: Optional[ctypes.CDLL] = None


def moe_grouped_supported(hidden: int, inter: int) -> bool:
    """Whether the grouped tensor-core expert products take these inner sizes (k16 steps, 16-byte rows)."""
    return hidden >= 16 and inter >= 16 and hidden % 16 == 0 and inter % 16 == 0


def moe_grouped_lib() -> ctypes.CDLL:
    global _moe_grouped
    with _lock:
        if _moe_grouped is None:
            import os

            defs = {}   # measurement knobs: the ring's slice width and depth (the source's defaults otherwise)
            for var, name in (("DRYFT_MOE_BK", "DRYFT_MOE_BK"), ("DRYFT_MOE_STAGES", "DRYFT_MOE_STAGES")):
                if os.environ.get(var):
                    defs[name] = int(os.environ[var])
            lib = _load(build.build_library("moe_grouped", ("moe_grouped.cu",), defs))
            lib.dryft_moe_grouped.argtypes = [_p, _p, _p, _p, _i, _i, _i, _i, _i, _p, _p, _p, _i, _p, _f, _f, _f, _p]
            lib.dryft_moe_grouped.restype = _i
            lib.dryft_moe_grouped_work_ints.argtypes = [_i, _i]
            lib.dryft_moe_grouped_work_ints.restype = _ll
            _moe_grouped = lib
        return _moe_grouped


def moe_grouped(h, w_gate_up, w_down, idx, y, gated: bool = True, in_w=None, limit: Optional[float] = None, alpha: float = 1.0,
                up_offset: float = 0.0) -> None:
    """``y[n*top + k] = expert idx[n, k] applied to h[n]`` (bfloat16) with the assignments sorted by expert on the device and
    both expert products as grouped tensor-core products (``csrc/moe_grouped.cu``: three launches, no host round trip).
    ``gated=False``: ``w_gate_up`` is ``[E, F, W]`` (no gate rows) and the activation is ``max(., 0)^2``.  With ``in_w [n, top]``
    (float32) each assignment's weight scales its expert's input and the activation is the clamped one of ``moe_rows``'s
    ``gate_up_clamp`` mode."""
    n, width = h.shape
    top = idx.shape[1]
    e, two_f, _ = w_gate_up.shape
    f = two_f // 2 if gated else two_f
    _need(h, "h", torch.bfloat16)
    _need(idx, "idx", torch.int32, (n, top))
    _need(w_gate_up, "w_gate_up", torch.bfloat16, (e, (2 if gated else 1) * f, width))
    _need(w_down, "w_down", torch.bfloat16, (e, width, f))
    _need(y, "y", torch.bfloat16, (n * top, width))
    if not moe_grouped_supported(width, f):
        raise KernelError(f"moe_grouped: inner sizes must be multiples of 16, got {width}, {f}")
    lib = moe_grouped_lib()
    work = torch.empty(int(lib.dryft_moe_grouped_work_ints(n * top, e)), dtype=torch.int32, device=h.device)
    act = torch.empty((n * top, f), dtype=torch.bfloat16, device=h.device)
    if in_w is not None:
        if not gated:
            raise KernelError("moe_grouped: weights on the experts' input go with gated experts")
        _need(in_w, "in_w", torch.float32, (n, top))
    _ok(lib.dryft_moe_grouped(_ptr(h), _ptr(w_gate_up), _ptr(w_down), _ptr(idx), n, top, e, width, f, _ptr(act), _ptr(y), _ptr(work),
                              2 if in_w is not None else int(gated), _ptr(in_w), float("inf") if limit is None else float(limit),
                              float(alpha), float(up_offset), _stream()), f"moe_grouped ({e} experts, {width} x {f})", n_kernels=3)


# ----------------------------------------------------------------------------- matrix products
def gemm_nt_f32(a, w, out) -> None:
    """``out[M,N] = a[M,K] @ w[N,K].T`` in true 32-bit."""
    m, k = a.shape
    n = w.shape[0]
    _need(a, "a", torch.float32)
    _need(w, "w", torch.float32, (n, k))
    _need(out, "out", torch.float32, (m, n))
    _ok(core().dryft_gemm_nt_f32(_ptr(a), k, _ptr(w), _ptr(out), n, m, n, k, _stream()), "gemm_nt_f32")


SMALL_M_LIMIT = 16  # rows the weight-streaming product takes
SS_STRIDE = 64  # floats per block in the sum-of-squares buffers of the fused decode products


def weighted_ahead_supported(k: int) -> bool:
    """Whether products over ``k`` inputs can take / leave activations weighted ahead (``xw_in`` / ``xw_out``)."""
    return k > 0 and k % 256 == 0


def small_m_ss_parts(n: int, k: int) -> int:
    """Blocks of sums of squares (64 floats each) that ``gemm_small_m(mode="residual")`` leaves for ``n`` outputs over
    ``k`` inputs: one per 16-row tile."""
    return (n + 15) // 16


def gemm_small_m(a, w, out, *, mode: str = "store", norm_w=None, ss_in=None, ss_parts: int = 0, eps: float = 0.0,
                 ss_out=None, pdl: bool = False, xw_in=None, next_w=None, xw_out=None) -> None:
    """``a[M,K] @ w[.,K].T`` for up to 16 rows (decode; K a multiple of 16): bfloat16 operands, 32-bit accumulation,
    every weight byte read once.  ``mode``:

    * ``"store"``: ``out[M,N]`` (bfloat16 or float32) receives the product, ``w`` is ``[N,K]``;
    * ``"residual"``: ``out`` is the residual stream ``x[M,N]``, updated in place ``x += product``; with
      ``ss_out`` ``[small_m_ss_parts(N, K), 64]`` float32 the per-row sums of squares of the new ``x`` are left
      there, one partial per tile of up to 16 columns;
    * ``"silu"``: ``w`` is ``[2N,K]`` (gate rows, then up rows) and ``out[M,N] = silu(gate) * up``.

    With ``norm_w`` ``[K]`` float32 the rows of ``a`` are RMS-normalised on the fly; ``ss_in``
    ``[ss_parts, 64]`` holds their sums of squares as an earlier ``"residual"`` product (or ``row_sumsq``)
    left them.  ``pdl`` launches the kernel as a programmatic dependent of the launch before it: its
    first weight requests overlap that launch's tail.

    The norm split over two launches (inner sizes that are multiples of 256 only, ``weighted_ahead_supported``):
    a ``"residual"`` product given the next norm's weight ``next_w`` ``[N]`` also leaves ``xw_out[M,N] =
    T(x * next_w)``; a product given such ``xw_in`` ``[M,K]`` (with ``ss_in``, ``eps``) multiplies it as plain
    activations and scales its sums by the norm's factor in the epilogue -- no prologue on its critical path."""
    m, k = a.shape
    _need(a, "a", torch.bfloat16)
    if xw_in is not None:
        if not weighted_ahead_supported(k):
            raise KernelError(f"gemm_small_m: activations weighted ahead need an inner size that is a multiple of 256, got {k}")
        _need(xw_in, "xw_in", torch.bfloat16, (m, k))
    if (next_w is None) != (xw_out is None):
        raise KernelError("gemm_small_m: next_w and xw_out go together")
    if xw_out is not None and (mode != "residual" or not weighted_ahead_supported(k)):
        raise KernelError("gemm_small_m: xw_out belongs to mode='residual' with an inner size that is a multiple of 256")
    if mode == "silu":
        n = w.shape[0] // 2
        _need(w, "w", torch.bfloat16, (2 * n, k))
        _need(out, "out", torch.bfloat16, (m, n))
        code = 3
    elif mode == "residual":
        n = w.shape[0]
        _need(w, "w", torch.bfloat16, (n, k))
        _need(out, "residual stream", torch.bfloat16, (m, n))
        code = 2
        if ss_out is not None:
            _need(ss_out, "ss_out", torch.float32)
            if ss_out.numel() < small_m_ss_parts(n, k) * SS_STRIDE:
                raise KernelError("gemm_small_m: ss_out too small (small_m_ss_parts(N, K) blocks of 64 floats are left)")
    elif mode == "store":
        n = w.shape[0]
        _need(w, "w", torch.bfloat16, (n, k))
        _need(out, "out", None, (m, n))
        if out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError(f"gemm_small_m: output must be bfloat16 or float32, got {out.dtype}")
        code = int(out.dtype == torch.float32)
    else:
        raise KernelError(f"gemm_small_m: unknown mode {mode!r}")
    if mode != "residual" and ss_out is not None:
        raise KernelError("gemm_small_m: ss_out belongs to mode='residual'")
    if norm_w is not None or xw_in is not None:
        if norm_w is not None:
            _need(norm_w, "norm_w", torch.float32, (k,))
        _need(ss_in, "ss_in", torch.float32)
        if ss_parts <= 0 or ss_in.numel() < ss_parts * SS_STRIDE:
            raise KernelError("gemm_small_m: ss_in does not hold ss_parts blocks")
    if xw_out is not None:
        _need(next_w, "next norm weight", torch.float32, (n,))
        _need(xw_out, "xw_out", torch.bfloat16, (m, n))
    if k % 256 == 0:  # the form compiled for this inner size: loops unrolled, offsets immediate
        lib = gemm_decode_lib(k)
        if xw_in is not None:
            rc = lib.dryft_gemm_decode(_ptr(xw_in), k, _ptr(w), _ptr(out), n, code, m, n, None, _ptr(ss_in), int(ss_parts),
                                       float(eps), _ptr(ss_out), int(pdl), 1, _ptr(next_w), _ptr(xw_out), _stream())
            if rc != UNSUPPORTED:
                _ok(rc, f"gemm_decode (M={m}, N={n}, K={k}, mode={mode}, activations weighted ahead)")
                return
            if norm_w is None:  # it refuses what does not fit its shared memory; with norm_w the plain form takes over
                _ok(rc, f"gemm_decode (M={m}, N={n}, K={k}, mode={mode}, activations weighted ahead; give norm_w for the other form)")
        rc = lib.dryft_gemm_decode(_ptr(a), k, _ptr(w), _ptr(out), n, code, m, n, _ptr(norm_w), _ptr(ss_in), int(ss_parts),
                                   float(eps), _ptr(ss_out), int(pdl), 0, _ptr(next_w), _ptr(xw_out), _stream())
        if rc != UNSUPPORTED or xw_out is not None or ss_out is not None:
            # the general form below cannot leave xw_out, and leaves another number of blocks of sums of squares
            _ok(rc, f"gemm_decode (M={m}, N={n}, K={k}, mode={mode})")
            return
    _ok(core().dryft_gemm_small_m(_ptr(a), k, _ptr(w), _ptr(out), n, code, m, n, k, _ptr(norm_w), _ptr(ss_in),
                                  int(ss_parts), float(eps), _ptr(ss_out), int(pdl), _stream()),
        f"gemm_small_m (M={m}, N={n}, K={k}, mode={mode})")


STREAM_M_LIMIT = 64


def gemm_stream_supported(m: int, k: int) -> bool:
    return 0 < m <= STREAM_M_LIMIT and k > 0 and k % 64 == 0


def gemm_stream_ss_parts(n_out: int, k_in: int) -> int:
    """Blocks of sums of squares that ``gemm_stream(mode="residual")`` leaves in ``ss_out``."""
    return int(gemm_stream_lib().dryft_gemm_stream_ss_parts(int(n_out), int(k_in)))


def gemm_stream(a, w, out, *, mode: str = "store", norm_w=None, ss_in=None, ss_parts: int = 0, eps: float = 0.0,
                ss_out=None, pdl: bool = False) -> None:
    """``gemm_small_m``'s contract for up to 64 rows, on tcgen05 with the weights streamed by TMA through a
    shared-memory ring, the work cut evenly over the SMs and tiles that two blocks share summed in block order.
    ``ss_out`` must hold ``gemm_stream_ss_parts(N, K)`` blocks of 64 floats."""
    m, k = a.shape
    _need(a, "a", torch.bfloat16)
    if not gemm_stream_supported(m, k):
        raise KernelError(f"gemm_stream takes 1..{STREAM_M_LIMIT} rows and inner sizes that are multiples of 64, got M={m}, K={k}")
    code = {"store": 1 if out.dtype == torch.float32 else 0, "residual": 2, "silu": 3}.get(mode)
    if code is None:
        raise KernelError(f"gemm_stream: unknown mode {mode!r}")
    rows = w.shape[0]
    n = rows // 2 if mode == "silu" else rows
    _need(w, "w", torch.bfloat16, (2 * n if mode == "silu" else n, k))
    _need(out, "out", torch.float32 if code == 1 else torch.bfloat16, (m, n))
    if n > (1 << 16) * 64:
        raise KernelError(f"gemm_stream: {n} outputs are more than its ticket counters cover")
    if norm_w is not None:
        if mode == "residual":
            raise KernelError("gemm_stream: a residual product takes plain activations")
        _need(norm_w, "norm weight", torch.float32, (k,))
        _need(ss_in, "ss_in", torch.float32)
        if ss_parts <= 0 or ss_in.numel() < ss_parts * SS_STRIDE:
            raise KernelError("gemm_stream: ss_in does not hold ss_parts blocks")
    if ss_out is not None:
        if mode != "residual":
            raise KernelError("gemm_stream: ss_out belongs to mode='residual'")
        _need(ss_out, "ss_out", torch.float32)
        if ss_out.numel() < gemm_stream_ss_parts(n, k) * SS_STRIDE:
            raise KernelError("gemm_stream: ss_out too small")
    ws, tk = gemm_stream_scratch(a.device)
    _ok(gemm_stream_lib().dryft_gemm_stream(_ptr(a), k, _ptr(w), _ptr(out), n, code, m, n, k, _ptr(norm_w), _ptr(ss_in),
                                            int(ss_parts), float(eps), _ptr(ss_out), int(pdl), _ptr(error_flag(a.device)),
                                            _ptr(ws), _ptr(tk), _stream()),
        f"gemm_stream (M={m}, N={n}, K={k}, mode={mode})")


SMALL_M_CUT_BYTES = 100 * 1024  # the shared-memory cut that csrc/gemm_decode.cu asks for (CARVEOUT_BYTES)


def small_m_staged_bytes(m: int, k: int) -> int:
    """Shared memory of one block of the per-size decode product with the norm on the way in (csrc/gemm_decode.cu,
    ``launch3``): two groups' partial sums or the norm's weight, 64 factors, the ``m`` rows and a row of zeros, one
    reserved KB."""
    mp = 8 if m <= 8 else 16
    head = (max(2 * 8 * 16 * (mp + 1) * 4, k * 2) + 15) // 16 * 16   # two groups' partial sums
    rows = m + 1 if m < mp else mp
    return head + 256 + rows * (k + 32) * 2 + 1024


def fused_rows_supported(m: int, k: int, small_m_max: int, stream_m_max: int, normed: bool = False) -> bool:
    """Whether ``fused_product`` takes ``m`` rows over ``k`` inputs: the register-streaming product up to
    ``small_m_max`` rows, the tcgen05 one up to ``stream_m_max``.  ``normed``: the product has the norm on its way
    in, so its rows stay in shared memory; above 8 rows that is taken only for widths whose 16 staged rows keep
    a block under the cut that leaves L1 large enough for the weights in flight.  Measured at 9 to 16 rows:
    width 2,560: 2.38-2.40 ms a step against 2.74-2.77 ms with the library's products; width 4,096 (ten rows
    fit): 4.18 against 3.86 ms; width 5,120: 16.4 against 13.2 ms."""
    if m <= min(small_m_max, SMALL_M_LIMIT):
        if m > 8 and normed and k % 256 == 0 and small_m_staged_bytes(16, k) > SMALL_M_CUT_BYTES:
            return False
        return k % 16 == 0
    return m <= min(stream_m_max, STREAM_M_LIMIT) and gemm_stream_supported(m, k)


def fused_ss_parts(m: int, n: int, k: int, small_m_max: int) -> int:
    """Blocks of sums of squares that ``fused_product(mode="residual")`` of these sizes leaves in ``ss_out``."""
    if m <= min(small_m_max, SMALL_M_LIMIT):
        return small_m_ss_parts(n, k)
    return gemm_stream_ss_parts(n, k)


def fused_product(a, w, out, *, small_m_max: int, **kw) -> None:
    """A decode product with its norm / residual / SiLU*mul fused in, by the kernel that suits the row count:
    ``gemm_small_m`` (weights streamed through registers into mma.sync) up to ``small_m_max`` rows, ``gemm_stream``
    (TMA ring, tcgen05, even cut over the SMs) above.  Activations weighted ahead (``xw_in`` / ``xw_out``) belong
    to the former only."""
    if a.shape[0] <= min(small_m_max, SMALL_M_LIMIT):
        gemm_small_m(a, w, out, **kw)
        return
    if kw.get("xw_in") is not None or kw.get("xw_out") is not None:
        raise KernelError("fused_product: activations weighted ahead are not taken above small_m_max rows")
    kw = {k_: v for k_, v in kw.items() if k_ not in ("xw_in", "xw_out", "next_w")}
    gemm_stream(a, w, out, **kw)


def row_sumsq(x, ss, norm_w=None, xw_out=None) -> None:
    """``ss[m] = sum(x[m]^2)`` for up to 64 rows of bfloat16 ``x``: one block of sums of squares.  With a norm
    weight it also leaves ``xw_out = T(x * norm_w)`` for a product that takes activations weighted ahead."""
    rows, hidden = x.shape
    _need(x, "x", torch.bfloat16)
    _need(ss, "ss", torch.float32)
    if ss.numel() < SS_STRIDE:
        raise KernelError("row_sumsq: ss holds fewer than 64 floats")
    if (norm_w is None) != (xw_out is None):
        raise KernelError("row_sumsq: norm_w and xw_out go together")
    if xw_out is not None:
        _need(norm_w, "norm weight", torch.float32, (hidden,))
        _need(xw_out, "xw_out", torch.bfloat16, (rows, hidden))
    _ok(core().dryft_row_sumsq(_ptr(x), rows, hidden, _ptr(ss), _ptr(norm_w), _ptr(xw_out), _stream()), "row_sumsq")


# ----------------------------------------------------------------------------- token choice
def argmax_rows(logits, out, row_slot=None, last_token=None) -> None:
    rows, vocab = logits.shape
    _need(logits, "logits", torch.float32)
    _need(out, "chosen tokens", torch.int32)
    if out.numel() < rows:
        raise KernelError("argmax_rows: output shorter than the rows")
    if row_slot is not None:
        _need(row_slot, "row_slot", torch.int32)
        _need(last_token, "last_token", torch.int32)
    _ok(core().dryft_argmax_rows(_ptr(logits), rows, vocab, vocab, _ptr(out), _ptr(row_slot), _ptr(last_token), _stream()),
        "argmax_rows")


def sample_rows(logits, temperature: float, top_k: int, seed: int, row_seq, row_step, out, row_slot=None, last_token=None,
                step_base: int = 0) -> None:
    """Row r draws with uniform(seed, row_seq[r] (or r), step_base + row_step[r] (or 0))."""
    rows, vocab = logits.shape
    _need(logits, "logits", torch.float32)
    _need(out, "chosen tokens", torch.int32)
    if not temperature > 0.0:
        raise KernelError("sample_rows: temperature must be positive (use argmax_rows for greedy)")
    for t, nm in ((row_seq, "row_seq"), (row_step, "row_step")):
        if t is None:
            continue
        _need(t, nm, torch.int32)
        if t.numel() < rows:
            raise KernelError(f"sample_rows: {nm} shorter than the rows")
    if row_slot is not None:
        _need(row_slot, "row_slot", torch.int32)
        _need(last_token, "last_token", torch.int32)
    _ok(core().dryft_sample_rows(_ptr(logits), rows, vocab, vocab, float(temperature), int(top_k), int(seed) & (2**64 - 1),
                                 _ptr(row_seq), _ptr(row_step), int(step_base), _ptr(out), _ptr(row_slot), _ptr(last_token),
                                 _stream()), "sample_rows")


# ----------------------------------------------------------------------------- libraries built only for models that use them
_single: Dict[str, ctypes.CDLL] = {}


def _single_lib(name: str, protos: Dict[str, list]) -> ctypes.CDLL:
    """A library made of one source file ``<name>.cu``, compiled the first time a model needs it."""
    with _lock:
        lib = _single.get(name)
        if lib is None:
            lib = _load(build.build_library(name, (name + ".cu",)))
            for fn, argtypes in protos.items():
                getattr(lib, fn).argtypes = argtypes
                getattr(lib, fn).restype = _i
            _single[name] = lib
        return lib


def stream_hc_lib() -> ctypes.CDLL:
    """Several residual streams joined by small matrices, the embedding that starts them, the clamped gated activation."""
    return _single_lib("stream_hc", {
        "dryft_embed_pair_norm": [_i, _p, _p, _p, _p, _p, _p, _i, _ll, _ll, _f, _p, _f, _p, _i, _i, _i, _p, _p],
        "dryft_seq_last_token": [_p, _p, _i, _p, _p],
        "dryft_hc_step": [_i, _p, _i, _p, _i, _p, _p, _p, _f, _p, _p, _f, _p, _p, _i, _i, _p],
        "dryft_glu_clamp": [_i, _p, _p, _i, _i, _f, _i, _f, _f, _p],
    })


def recurrent_lib() -> ctypes.CDLL:
    """Mixers with a fixed-size 32-bit state per sequence: retention, gated linear recurrence."""
    return _single_lib("recurrent", {
        "dryft_retention_chunked": [_i, _p, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _f, _f, _p],
        "dryft_retention_chunk_tokens": [],
        "dryft_retention_scan": [_i, _p, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _i, _p, _p, _p, _i, _i, _i, _i, _f, _f, _p],
        "dryft_rglru_gates": [_i, _p, _i, _i, _p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _f, _p, _p, _i, _i, _i, _p],
        "dryft_rglru_scan": [_i, _p, _i, _i, _p, _i, _p, _p, _p, _p, _p, _p, _p, _i, _p, _i, _i, _p],
    })


def latent_attn_lib() -> ctypes.CDLL:
    """Attention over cached low-rank latents."""
    return _single_lib("latent_attn", {
        "dryft_latent_prep": [_i, _p, _i, _i, _i, _p, _i, _i, _i, _p, _f, _p, _p, _i, _p, _p, _p, _p, _p, _i, _i, _p, _i, _p],
        "dryft_latent_scratch_table": [_p, _p, _i, _p, _i, _i, _p],
        "dryft_latent_expand_store": [_i, _p, _p, _i, _i, _p, _i, _i, _p, _p, _i, _p, _p, _p, _i, _i, _p, _p, _p, _i, _i, _i, _i, _i, _p],
        "dryft_head_gate_rows": [_i, _p, _i, _p, _i, _p, _i, _i, _i, _p],
        "dryft_latent_fold_q": [_i, _p, _i, _p, _p, _i, _i, _i, _i, _p],
        "dryft_latent_unfold_o": [_i, _p, _p, _p, _i, _p, _i, _i, _i, _i, _p],
        "dryft_latent_attn_rows": [_i, _p, _p, _i, _i, _p, _p, _i, _i, _p, _p, _p, _p, _i, _p, _p, _i, _i, _i, _i, _i, _f, _i, _p, _p],
        "dryft_head_gate": [_i, _p, _p, _i, _p, _i, _i, _i, _p],
    })


# ----------------------------------------------------------------------------- streams joined by small matrices
HC_MAX_STREAMS = 8


def embed_pair_norm(tokens, tok_slot, tok_pos, table, x32, *, scale: float = 1.0, pair_table=None, buckets: int = 0,
                    mul_prev: int = 0, mul_cur: int = 0, prev_state=None, norm_w=None, eps: float = 0.0, err=None) -> None:
    """``x32[n] = norm(table[tokens[n]] * scale + pair_table[row]) * norm_w`` (32-bit), ``row`` hashed from the token and the
    one before it in its sequence (``prev_state[slot]`` for the first token a sequence brings in a step; the table's row
    ``buckets`` for a sequence's first token).  Without ``pair_table`` nothing is added, without ``norm_w`` nothing normed."""
    n, width = x32.shape
    _need(x32, "stream", torch.float32)
    for t, nm in ((tokens, "tokens"), (tok_slot, "tok_slot"), (tok_pos, "tok_pos")):
        _need(t, nm, torch.int32)
        if t.numel() < n:
            raise KernelError(f"embed_pair_norm: {nm} shorter than the rows")
    _need(table, "embedding table", None, (None, width))
    if pair_table is not None:
        _need(pair_table, "pair table", table.dtype, (buckets + 1, width))
        _need(prev_state, "prev_state", torch.int32)
    if norm_w is not None:
        _need(norm_w, "norm weight", torch.float32, (width,))
    if err is not None:
        _need(err, "err", torch.int32)
    _ok(stream_hc_lib().dryft_embed_pair_norm(_act(table, "embedding table"), _ptr(tokens), _ptr(tok_slot), _ptr(tok_pos),
                                              _ptr(prev_state), _ptr(table), _ptr(pair_table), int(buckets), int(mul_prev),
                                              int(mul_cur), float(scale), _ptr(norm_w), float(eps), _ptr(x32), n, width,
                                              table.shape[0], _ptr(err), _stream()), f"embed_pair_norm (width {width})")


def seq_last_token(tokens, tok_slot, n: int, prev_state) -> None:
    """``prev_state[slot] =`` the last token each sequence brought in this step."""
    for t, nm in ((tokens, "tokens"), (tok_slot, "tok_slot"), (prev_state, "prev_state")):
        _need(t, nm, torch.int32)
    _ok(stream_hc_lib().dryft_seq_last_token(_ptr(tokens), _ptr(tok_slot), n, _ptr(prev_state), _stream()), "seq_last_token")


def hc_step(x_in, n_streams: int, *, x_out=None, y=None, mix=None, outw=None, mult: float = 1.0, inw=None, norm_w=None,
            eps: float = 0.0, rows=None, h=None) -> None:
    """One joint of a residual stream held as ``n_streams`` 32-bit copies.  ``x_in`` is ``[n, n_streams, W]`` or ``[n, W]``
    (one copy standing for all).  With ``y [n, W]``: ``x'_t = sum_s mix[s, t] x_s + mult * outw[t] * y``; written to
    ``x_out [n, n_streams, W]`` if given (may be ``x_in``).  With ``inw``: ``h = T(rmsnorm(sum_t inw[t] x'_t) * norm_w)``;
    with ``rows`` (int32) ``h[r]`` is made from row ``rows[r]`` (``x_out`` must then be left out)."""
    _need(x_in, "streams", torch.float32)
    if x_in.dim() == 3:
        n, s_in, width = x_in.shape
    elif x_in.dim() == 2:
        (n, width), s_in = x_in.shape, 1
    else:
        raise KernelError(f"hc_step: streams are [n, S, W] or [n, W], got {tuple(x_in.shape)}")
    if not 1 <= n_streams <= HC_MAX_STREAMS or s_in not in (1, n_streams):
        raise KernelError(f"hc_step: {n_streams} streams (1..{HC_MAX_STREAMS}) against an input of {s_in}")
    if x_out is not None:
        if rows is not None:
            raise KernelError("hc_step: gathered rows are not written back")
        _need(x_out, "x_out", torch.float32, (n, n_streams, width))
    act = None
    if y is not None:
        _need(y, "y", None, (n, width))
        _need(mix, "mix", torch.float32, (n_streams, n_streams))
        _need(outw, "outw", torch.float32, (n_streams,))
        act = y
    n_rows = n
    if inw is not None:
        _need(inw, "inw", torch.float32, (n_streams,))
        _need(norm_w, "norm weight", torch.float32, (width,))
        if rows is not None:
            _need(rows, "rows", torch.int32)
            n_rows = h.shape[0]
            if rows.numel() < n_rows:
                raise KernelError("hc_step: fewer row indices than output rows")
        _need(h, "h", None, (n_rows, width))
        if act is not None and h.dtype != act.dtype:
            raise KernelError(f"hc_step: y is {act.dtype}, h is {h.dtype}")
        act = h
    elif rows is not None:
        raise KernelError("hc_step: rows belong to the norm's output")
    if act is None:
        raise KernelError("hc_step: nothing to do (neither y nor inw)")
    _ok(stream_hc_lib().dryft_hc_step(_act(act, "activations"), _ptr(x_in), s_in, _ptr(x_out), n_streams, _ptr(y), _ptr(mix), _ptr(outw),
                                      float(mult), _ptr(inw), _ptr(norm_w), float(eps), _ptr(rows), _ptr(h), n_rows, width, _stream()),
        f"hc_step ({n_streams} streams, width {width})")


def glu_clamp(gate_up, out, limit: Optional[float], alpha: float, up_offset: float) -> None:
    """``out = g * sigmoid(alpha * g) * (u + up_offset)`` with ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``
    (no clamping when ``limit`` is None); ``gate_up [rows, 2F]`` holds the gate columns first."""
    rows, two_f = gate_up.shape
    _need(gate_up, "gate_up")
    if two_f % 2:
        raise KernelError(f"glu_clamp: fused gate|up width must be even, got {two_f}")
    _need(out, "glu_clamp output", gate_up.dtype, (rows, two_f // 2))
    _ok(stream_hc_lib().dryft_glu_clamp(_act(gate_up, "gate_up"), _ptr(gate_up), _ptr(out), rows, two_f // 2,
                                        float(limit if limit is not None else 0.0), int(limit is not None), float(alpha),
                                        float(up_offset), _stream()), "glu_clamp")


# ----------------------------------------------------------------------------- recurrent mixers
def _freq_lo(inv_freq_lo, rot: int):
    if inv_freq_lo is not None and rot:
        _need(inv_freq_lo, "inv_freq_lo", torch.float32, (rot // 2,))
        return inv_freq_lo
    return None


RETENTION_CHUNKED_MAX_VDIM = 512   # value sizes the chunked form holds in a thread's registers


def retention_scan(proj, offsets, cu_q, seq_slot, tok_pos, inv_freq, rot: int, decay, state, out, n_seqs: int, heads: int,
                   dim: int, vdim: int, k_scale: float, eps: float, inv_freq_lo=None, chunked: bool = False) -> None:
    """``inv_freq_lo`` (optional, here and in the latent attention wrappers): the part of each frequency that its 32-bit
    value drops; with it the angles are as exact as the pair.

    Retention over the step's tokens from and to ``state [slots, heads, dim, vdim]`` (float32).  ``proj [n, ld]`` holds
    q | k | v | g at the column ``offsets`` (4 ints); ``out [n, heads * vdim]``; ``decay [heads]`` float64.  ``chunked``:
    the form for steps of many tokens (the same result up to rounding; token by token otherwise)."""
    n, ld = proj.shape
    _need(proj, "proj")
    q_off, k_off, v_off, g_off = (int(o) for o in offsets)
    if max(q_off + heads * dim, k_off + heads * dim, v_off + heads * vdim, g_off + heads * vdim) > ld:
        raise KernelError("retention_scan: column offsets outside the projection row")
    for t, nm in ((cu_q, "cu_q"), (seq_slot, "seq_slot"), (tok_pos, "tok_pos")):
        _need(t, nm, torch.int32)
    if rot:
        _need(inv_freq, "inv_freq", torch.float32, (rot // 2,))
    _need(decay, "decay", torch.float64, (heads,))
    _need(state, "state", torch.float32, (None, heads, dim, vdim))
    _need(out, "out", proj.dtype, (n, heads * vdim))
    if chunked and vdim <= RETENTION_CHUNKED_MAX_VDIM:
        # steps of many tokens: chunk states, their prefix, chunk outputs (three launches, the work spread over chunks)
        lib = recurrent_lib()
        ch = int(lib.dryft_retention_chunk_tokens())
        sbuf = torch.empty((n // ch + n_seqs) * heads * dim * vdim, dtype=torch.float32, device=proj.device)
        rc = lib.dryft_retention_chunked(_act(proj, "proj"), _ptr(proj), ld, q_off, k_off, v_off, g_off, _ptr(cu_q), _ptr(seq_slot),
                                         _ptr(tok_pos), _ptr(inv_freq), _ptr(_freq_lo(inv_freq_lo, rot)), int(rot), _ptr(decay), _ptr(state),
                                         _ptr(sbuf), _ptr(out), n, n_seqs, heads, dim, vdim, float(k_scale), float(eps), _stream())
        if rc != UNSUPPORTED:   # sizes whose chunk does not fit its shared memory are walked token by token below
            _ok(rc, f"retention_chunked ({heads} heads of {dim} x {vdim})", n_kernels=3)
            return
    _ok(recurrent_lib().dryft_retention_scan(_act(proj, "proj"), _ptr(proj), ld, q_off, k_off, v_off, g_off, _ptr(cu_q), _ptr(seq_slot),
                                             _ptr(tok_pos), _ptr(inv_freq), _ptr(_freq_lo(inv_freq_lo, rot)), int(rot), _ptr(decay), _ptr(state), _ptr(out), n_seqs,
                                             heads, dim, vdim, float(k_scale), float(eps), _stream()),
        f"retention_scan ({heads} heads of {dim} x {vdim})")


def rglru(proj, y_off: int, x_off: int, y_bias, x_bias, cu_q, seq_slot, tok_slot, conv_w, conv_b, w_gates, b_a, b_i, sp_lam,
          c_mult: float, state, tail, out, n_seqs: int, n_blocks: int) -> None:
    """The gated linear recurrence over ``C`` channels: ``proj [n, ld]`` holds the gelu branch at ``y_off`` and the recurrent
    branch at ``x_off`` (biases not added yet); ``conv_w [C, taps]``; ``w_gates [blocks, C/blocks (in), 2, C/blocks (out)]``
    (recurrence gate, input gate); ``state [slots, C]`` and ``tail [slots, taps-1, C]`` float32; ``out [n, C]``.  Two launches."""
    n, ld = proj.shape
    c, taps = conv_w.shape
    _need(proj, "proj")
    if c % n_blocks or max(y_off, x_off) + c > ld:
        raise KernelError(f"rglru: {c} channels in {n_blocks} groups, row of {ld}")
    nb = c // n_blocks
    for t, nm, shp in ((y_bias, "y_bias", (c,)), (x_bias, "x_bias", (c,)), (conv_w, "conv_w", (c, taps)), (conv_b, "conv_b", (c,)),
                       (w_gates, "w_gates", (n_blocks, nb, 2, nb)), (b_a, "b_a", (c,)), (b_i, "b_i", (c,)), (sp_lam, "sp_lam", (c,)),
                       (state, "state", (None, c))):
        _need(t, nm, torch.float32, shp)
    if taps > 1:
        _need(tail, "tail", torch.float32, (state.shape[0], taps - 1, c))
    for t, nm in ((cu_q, "cu_q"), (seq_slot, "seq_slot"), (tok_slot, "tok_slot")):
        _need(t, nm, torch.int32)
    _need(out, "out", proj.dtype, (n, c))
    a = torch.empty((n, c), dtype=torch.float32, device=proj.device)
    b = torch.empty((n, c), dtype=torch.float32, device=proj.device)
    lib = recurrent_lib()
    is_bf16 = _act(proj, "proj")
    _ok(lib.dryft_rglru_gates(is_bf16, _ptr(proj), ld, int(x_off), _ptr(x_bias), _ptr(tok_slot), _ptr(conv_w), _ptr(conv_b), taps,
                              _ptr(tail if taps > 1 else None), _ptr(w_gates), _ptr(b_a), _ptr(b_i), _ptr(sp_lam), float(c_mult),
                              _ptr(a), _ptr(b), n, c, n_blocks, _stream()), f"rglru_gates ({c} channels, {n_blocks} groups)")
    _ok(lib.dryft_rglru_scan(is_bf16, _ptr(proj), ld, int(y_off), _ptr(y_bias), int(x_off), _ptr(x_bias), _ptr(cu_q), _ptr(seq_slot),
                             _ptr(a), _ptr(b), _ptr(state), _ptr(tail if taps > 1 else None), taps, _ptr(out), n_seqs, c, _stream()),
        f"rglru_scan ({c} channels)")


# ----------------------------------------------------------------------------- attention over cached latents
def latent_prep(proj, dq_off: int, q_rank: int, w_q, dkv_off: int, kv_rank: int, rot: int, w_kv, eps: float, inv_freq,
                interleaved: bool, tok_slot, tok_pos, cq, k_pages, page_table, inv_freq_lo=None, c_out=None) -> None:
    """Normalise the query latent into ``cq [n, q_rank]``; normalise the key/value latent, rotate the shared key part and
    write ``[c | k_rot]`` into the paged cache ``k_pages [pages, 1, page, kv_rank + rot]`` at each token's (slot, position)."""
    n, ld = proj.shape
    _need(proj, "proj")
    if dq_off + q_rank > ld or dkv_off + kv_rank + rot > ld:
        raise KernelError("latent_prep: column ranges outside the projection row")
    _need(w_q, "w_q", torch.float32, (q_rank,))
    _need(w_kv, "w_kv", torch.float32, (kv_rank,))
    if rot:
        _need(inv_freq, "inv_freq", torch.float32, (rot // 2,))
    _need(tok_slot, "tok_slot", torch.int32)
    _need(tok_pos, "tok_pos", torch.int32)
    _need(cq, "cq", proj.dtype, (n, q_rank))
    _need(k_pages, "k_pages", proj.dtype, (None, 1, None, kv_rank + rot))
    _need(page_table, "page_table", torch.int32)
    if c_out is not None:   # the normalised key/value latent as rows too
        _need(c_out, "c_out", proj.dtype, (n, kv_rank))
    _ok(latent_attn_lib().dryft_latent_prep(_act(proj, "proj"), _ptr(proj), ld, int(dq_off), q_rank, _ptr(w_q), int(dkv_off), kv_rank,
                                            rot, _ptr(w_kv), float(eps), _ptr(inv_freq), _ptr(_freq_lo(inv_freq_lo, rot)), int(interleaved), _ptr(tok_slot),
                                            _ptr(tok_pos), _ptr(cq), _ptr(k_pages), _ptr(page_table), page_table.shape[1],
                                            k_pages.shape[2], _ptr(c_out), n, _stream()), "latent_prep")


def latent_attn_rows(q_lat, q, q_rot_off: int, k_pages, page_table, tok_slot, tok_pos, inv_freq, interleaved: bool, o_lat,
                     kv_rank: int, rot: int, scale: float, window: Optional[int], inv_freq_lo=None, n_splits: int = 1, sink=None) -> None:
    """``o_lat [H, n, kv_rank]``: softmax attention of ``q_lat [H, n, kv_rank]`` (float32, the key matrices folded in) and the
    rotated part of ``q [n, H, q_stride]`` (at ``q_rot_off``, rotated here) over the cached rows ``[c | k_rot]``.
    ``n_splits``: blocks that share each token's visible keys (whole tiles of 32 keys each).  ``sink [H]`` (float32): the
    denominator of head ``h`` also holds ``exp(sink[h])``, which has no key and no value and is not scaled."""
    n_heads, n, _ = q_lat.shape
    if sink is not None:
        _need(sink, "sink", torch.float32, (n_heads,))
    _need(q_lat, "q_lat", torch.float32, (n_heads, n, kv_rank))
    _need(q, "q", k_pages.dtype, (n, n_heads, None))
    if q_rot_off + rot > q.shape[2]:
        raise KernelError("latent_attn_rows: the rotated part lies outside the query rows")
    _need(k_pages, "k_pages", None, (None, 1, None, kv_rank + rot))
    for t, nm in ((page_table, "page_table"), (tok_slot, "tok_slot"), (tok_pos, "tok_pos")):
        _need(t, nm, torch.int32)
    if rot:
        _need(inv_freq, "inv_freq", torch.float32, (rot // 2,))
    _need(o_lat, "o_lat", k_pages.dtype, (n_heads, n, kv_rank))
    part = None
    if n_splits > 1:   # each split's (max, sum, weighted sum), joined by a second launch
        part = torch.empty(n * n_heads * n_splits * (kv_rank + 2), dtype=torch.float32, device=o_lat.device)
    _ok(latent_attn_lib().dryft_latent_attn_rows(_act(k_pages, "k_pages"), _ptr(q_lat), _ptr(q), q.shape[2], int(q_rot_off), _ptr(k_pages),
                                                 _ptr(page_table), page_table.shape[1], k_pages.shape[2], _ptr(tok_slot), _ptr(tok_pos),
                                                 _ptr(inv_freq), _ptr(_freq_lo(inv_freq_lo, rot)), int(interleaved), _ptr(o_lat), _ptr(part), int(n_splits),
                                                 n, n_heads, kv_rank, rot, float(scale), int(window or 0), _ptr(sink), _stream()),
        f"latent_attn_rows (rank {kv_rank}, rotated {rot})", n_kernels=2 if n_splits > 1 else 1)


def latent_expand_store(q, kv, v_off: int, proj, krot_off: int, inv_freq, interleaved: bool, cu_q, seq_slot, n_seqs: int, tok_slot,
                        tok_pos, table, q_out, k_pages, v_pages, dim: int, rot: int, vdim: int, inv_freq_lo=None) -> None:
    """For a step whose sequences all start at position 0: pages of the step's own (``table [slots, pages]`` is filled
    here) receive per-head keys ``[k_plain | rotated shared part]`` and values ``[v | zeros]`` of head size ``dim + rot``;
    ``q_out [n, H, dim + rot]`` receives the queries with their rotated part rotated.  ``q [n, H, dim + rot]``,
    ``kv [n, >= H*dim + H*vdim]`` (keys' unrotated parts at column 0, values at ``v_off``), ``proj`` holds the shared key part
    at ``krot_off``.  Two launches."""
    n, n_heads, hd = q.shape
    _need(q, "q")
    if hd != dim + rot or vdim > hd:
        raise KernelError(f"latent_expand_store: head size {hd} against {dim} + {rot}, values of {vdim}")
    _need(kv, "kv", q.dtype)
    _need(proj, "proj", q.dtype)
    if kv.dim() != 2 or kv.shape[0] < n or kv.shape[1] < max(n_heads * dim, v_off + n_heads * vdim) or krot_off + rot > proj.shape[1]:
        raise KernelError("latent_expand_store: column ranges outside the rows")
    page = k_pages.shape[2]
    _need(q_out, "q_out", q.dtype, (n, n_heads, hd))
    _need(k_pages, "k_pages", q.dtype, (None, n_heads, page, hd))
    _need(v_pages, "v_pages", q.dtype, tuple(k_pages.shape))
    for t, nm in ((cu_q, "cu_q"), (seq_slot, "seq_slot"), (tok_slot, "tok_slot"), (tok_pos, "tok_pos"), (table, "table")):
        _need(t, nm, torch.int32)
    if rot:
        _need(inv_freq, "inv_freq", torch.float32, (rot // 2,))
    if k_pages.shape[0] < n // page + n_seqs or table.shape[1] < (n + page - 1) // page:
        raise KernelError("latent_expand_store: too few pages for the step")
    lib = latent_attn_lib()
    _ok(lib.dryft_latent_scratch_table(_ptr(cu_q), _ptr(seq_slot), n_seqs, _ptr(table), table.shape[1], page, _stream()),
        "latent_scratch_table")
    _ok(lib.dryft_latent_expand_store(_act(q, "q"), _ptr(q), _ptr(kv), kv.shape[1], int(v_off), _ptr(proj), proj.shape[1], int(krot_off),
                                      _ptr(inv_freq), _ptr(_freq_lo(inv_freq_lo, rot)), int(interleaved), _ptr(tok_slot), _ptr(tok_pos),
                                      _ptr(table), table.shape[1], page, _ptr(q_out), _ptr(k_pages), _ptr(v_pages), n, n_heads, dim, rot,
                                      vdim, _stream()), "latent_expand_store")


def head_gate_rows(o, gate, gate_col: int, out, n_heads: int, vdim: int) -> None:
    """``out[n, h*V + v] = T(o[n, h*hd + v] * sigmoid(gate[n, gate_col + h]))`` for ``o [n, H*hd]`` (``gate`` None: no gate)."""
    n = o.shape[0]
    hd = o.shape[1] // n_heads
    _need(o, "o", None, (n, n_heads * hd))
    _need(out, "out", o.dtype, (n, n_heads * vdim))
    gate_ptr, gate_ld = None, 0
    if gate is not None:
        _need(gate, "gate", out.dtype)
        if gate.dim() != 2 or gate.shape[0] < n or gate.shape[1] < gate_col + n_heads:
            raise KernelError("head_gate_rows: gate columns outside the gate tensor")
        gate_ptr, gate_ld = ctypes.c_void_p(gate.data_ptr() + gate_col * gate.element_size()), gate.shape[1]
    _ok(latent_attn_lib().dryft_head_gate_rows(_act(out, "out"), _ptr(o), hd, gate_ptr, gate_ld, _ptr(out), n, n_heads, vdim, _stream()),
        "head_gate_rows")


def head_gate(o, gate, gate_col: int, out) -> None:
    """``out[n, h*V + v] = T(o[h, n, v] * sigmoid(gate[n, gate_col + h]))`` (``gate`` None: no gate); ``o`` float32."""
    n_heads, n, vdim = o.shape
    _need(o, "o", torch.float32)
    _need(out, "out", None, (n, n_heads * vdim))
    gate_ptr, gate_ld = None, 0
    if gate is not None:
        _need(gate, "gate", out.dtype)
        if gate.dim() != 2 or gate.shape[0] < n or gate.shape[1] < gate_col + n_heads:
            raise KernelError("head_gate: gate columns outside the gate tensor")
        gate_ptr, gate_ld = ctypes.c_void_p(gate.data_ptr() + gate_col * gate.element_size()), gate.shape[1]
    _ok(latent_attn_lib().dryft_head_gate(_act(out, "out"), _ptr(o), gate_ptr, gate_ld, _ptr(out), n, n_heads, vdim, _stream()),
        "head_gate")


def latent_fold_q(q, w_k, q_lat, dim: int) -> None:
    """``q_lat[h, n, :] = q[n, h, :dim] @ w_k[h]`` with ``w_k [H, dim, kv_rank]``; float32 result, sums in a fixed order."""
    n, n_heads, q_stride = q.shape
    kv_rank = w_k.shape[2]
    _need(q, "q")
    _need(w_k, "w_k", q.dtype, (n_heads, dim, kv_rank))
    _need(q_lat, "q_lat", torch.float32, (n_heads, n, kv_rank))
    if dim > q_stride:
        raise KernelError("latent_fold_q: the unrotated part lies outside the query rows")
    _ok(latent_attn_lib().dryft_latent_fold_q(_act(q, "q"), _ptr(q), q_stride, _ptr(w_k), _ptr(q_lat), n, n_heads, dim, kv_rank, _stream()),
        "latent_fold_q")


def latent_unfold_o(o_lat, w_v, gate, gate_col: int, out) -> None:
    """``out[n, h*V:(h+1)*V] = T(sigmoid(gate[n, gate_col + h]) * (o_lat[h, n] @ w_v[h]))`` with ``w_v [H, kv_rank, V]``
    (``gate`` None: no gate)."""
    n_heads, n, kv_rank = o_lat.shape
    vdim = w_v.shape[2]
    _need(o_lat, "o_lat")
    _need(w_v, "w_v", o_lat.dtype, (n_heads, kv_rank, vdim))
    _need(out, "out", o_lat.dtype, (n, n_heads * vdim))
    gate_ptr, gate_ld = None, 0
    if gate is not None:
        _need(gate, "gate", out.dtype)
        if gate.dim() != 2 or gate.shape[0] < n or gate.shape[1] < gate_col + n_heads:
            raise KernelError("latent_unfold_o: gate columns outside the gate tensor")
        gate_ptr, gate_ld = ctypes.c_void_p(gate.data_ptr() + gate_col * gate.element_size()), gate.shape[1]
    _ok(latent_attn_lib().dryft_latent_unfold_o(_act(out, "out"), _ptr(o_lat), _ptr(w_v), gate_ptr, gate_ld, _ptr(out), n, n_heads, kv_rank,
                                                vdim, _stream()), "latent_unfold_o")


# ----------------------------------------------------------------------------- a stream whose norm follows the sum
def rowops_lib() -> ctypes.CDLL:
    """Row-wise kernels around a 32-bit stream with the norm after the sum, and activations over whole rows."""
    return _single_lib("rowops", {
        "dryft_gated_postnorm": [_i, _p, _p, _i, _p, _p, _i, _p, _i, _p, _p, _f, _f, _p, _p, _i, _i, _p],
        "dryft_polynorm": [_i, _p, _i, _p, _f, _p, _i, _i, _p],
        "dryft_relu2": [_i, _p, _i, _p, _i, _i, _p],
        "dryft_gated_group_norm": [_i, _p, _p, _i, _p, _i, _f, _p, _i, _i, _p],
    })


def gated_postnorm(y, x32, norm_w, alpha: float, eps: float, h=None, *, gate=None, gate_b=None, wts=None, top: int = 0,
                   shared=None, shared_gate=None) -> None:
    """``v = alpha * x32 + g * (y [+ sigmoid(shared_gate) * shared])`` with ``g = sigmoid(gate + gate_b)`` (1 without a gate);
    ``x32 <- v / sqrt(mean(v^2) + eps) * norm_w`` in place and ``h <- x32`` in the activation type (if given).  With ``wts
    [n, top]``, ``y`` holds ``top`` rows per row of the stream and their weighted sum is formed first.  ``gate`` and
    ``shared_gate`` may be column slices of a product's output (rows ``gate.stride(0)`` apart)."""
    n, w = x32.shape
    _need(x32, "x32", torch.float32)
    _need(norm_w, "norm_w", torch.float32, (w,))
    is_bf16 = _act(y, "y")
    _need(y, "y", None, (n * top if top else n, w))
    if top:
        _need(wts, "wts", torch.float32, (n, top))
    if h is not None:
        _need(h, "h", y.dtype, (n, w))
    gl_ld = 0
    if gate is not None:
        if gate.dtype != y.dtype or gate.shape != (n, w) or gate.stride(1) != 1 or not gate.is_cuda:
            raise KernelError(f"gated_postnorm: gate logits {tuple(gate.shape)} {gate.dtype} against a stream {tuple(x32.shape)}")
        gl_ld = gate.stride(0)
        _need(gate_b, "gate_b", torch.float32, (w,))
    sg_ld = 0
    if shared is not None:
        _need(shared, "shared", y.dtype, (n, w))
        if shared_gate is not None:
            if shared_gate.dtype != y.dtype or shared_gate.shape[0] != n or not shared_gate.is_cuda:
                raise KernelError("gated_postnorm: the always-on expert's gate logits are one per token, in the activation type")
            sg_ld = shared_gate.stride(0)
    _ok(rowops_lib().dryft_gated_postnorm(is_bf16, _ptr(y), _ptr(wts if top else None), int(top), _ptr(shared), _ptr(shared_gate),
                                          sg_ld, _ptr(gate), gl_ld, _ptr(gate_b), _ptr(norm_w), float(alpha), float(eps), _ptr(x32),
                                          _ptr(h), n, w, _stream()), f"gated_postnorm (width {w})")


def polynorm(z, coef, eps: float, out) -> None:
    """``out = a N(z) + b N(z^2) + c N(z^3) + e`` over each row, ``N(u) = u / sqrt(mean(u^2) + eps)``, ``coef = [a, b, c, e]``."""
    n, f = z.shape
    if z.stride(1) != 1 or not z.is_cuda:
        raise KernelError("polynorm: rows must be contiguous and on the device")
    _need(coef, "coef", torch.float32, (4,))
    _need(out, "out", z.dtype, (n, f))
    _ok(rowops_lib().dryft_polynorm(_act(z, "z"), _ptr(z), z.stride(0), _ptr(coef), float(eps), _ptr(out), n, f, _stream()),
        f"polynorm ({f} values a row)")


def relu2(z, out) -> None:
    """``out = max(z, 0)^2``; ``z`` may be a column slice of a product's output."""
    n, f = out.shape
    if z.shape != (n, f) or z.stride(1) != 1 or not z.is_cuda or z.dtype != out.dtype:
        raise KernelError(f"relu2: input {tuple(z.shape)} {z.dtype} against output {tuple(out.shape)} {out.dtype}")
    _need(out, "out")
    _ok(rowops_lib().dryft_relu2(_act(z, "z"), _ptr(z), z.stride(0), _ptr(out), n, f, _stream()), "relu2")


def gated_group_norm(y, z, weight, parts: int, eps: float, out) -> None:
    """``v = y * silu(z)``; each of ``parts`` equal parts of a row divided by its own root mean square, times ``weight``.
    ``y [n, inner]`` float32, ``z`` float32 (a column slice is fine), ``out [n, inner]`` in the activation type."""
    n, inner = y.shape
    _need(y, "y", torch.float32)
    if z.dtype != torch.float32 or z.shape != (n, inner) or z.stride(1) != 1 or not z.is_cuda:
        raise KernelError(f"gated_group_norm: gate {tuple(z.shape)} {z.dtype} against {tuple(y.shape)}")
    _need(weight, "weight", torch.float32, (inner,))
    _need(out, "out", None, (n, inner))
    _ok(rowops_lib().dryft_gated_group_norm(_act(out, "out"), _ptr(y), _ptr(z), z.stride(0), _ptr(weight), int(parts), float(eps),
                                            _ptr(out), n, inner, _stream()), f"gated_group_norm ({inner} in {parts} parts)")


# ----------------------------------------------------------------------------- selective state-space mixer
SSM_MAX_STATE = 512    # state rows a head may have (a lane of the scan holds up to sixteen)
SSM_MAX_TAPS = 16


def ssm_lib() -> ctypes.CDLL:
    return _single_lib("ssm", {
        "dryft_ssm_conv": [_p, _i, _i, _i, _p, _p, _i, _p, _p, _i, _p, _p, _p, _i, _p],
        "dryft_ssm_scan": [_p, _i, _p, _i, _i, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p, _p, _p],
        "dryft_ssm_scan_chunked": [_p, _i, _p, _i, _i, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p],
    })


SSM_CHUNK_TOKENS = 128    # tokens a chunk of a many-token step walks in order (more for steps of more than 8,192 tokens)


def ssm_conv(proj, x_off: int, conv_w, conv_b, cu_q, seq_slot, n_seqs: int, tail, out, out_bf16=None) -> None:
    """``out[t, c] = silu(conv_b[c] + sum_j conv_w[c, j] * in[t - (taps-1) + j, c])`` over the ``C`` channels of ``proj [n, ld]``
    (float32) from column ``x_off``; inputs from before the step come from ``tail [slots, taps-1, C]``, which is then
    advanced.  Two launches (one when there is a single tap).  ``out_bf16``: the same values once more, rounded (the operand of
    a bfloat16 product that follows)."""
    n, ld = proj.shape
    c, taps = conv_w.shape
    _need(proj, "proj", torch.float32)
    _need(conv_w, "conv_w", torch.float32)
    _need(conv_b, "conv_b", torch.float32, (c,))
    _need(out, "out", torch.float32, (n, c))
    if out_bf16 is not None:
        _need(out_bf16, "out_bf16", torch.bfloat16, (n, c))
    if x_off < 0 or x_off + c > ld:
        raise KernelError(f"ssm_conv: {c} channels from column {x_off} of a row of {ld}")
    if taps > 1:
        _need(tail, "tail", torch.float32, (None, taps - 1, c))
    for t, nm in ((cu_q, "cu_q"), (seq_slot, "seq_slot")):
        _need(t, nm, torch.int32)
    _ok(ssm_lib().dryft_ssm_conv(_ptr(proj), ld, int(x_off), c, _ptr(cu_q), _ptr(seq_slot), int(n_seqs), _ptr(conv_w), _ptr(conv_b),
                                 taps, _ptr(tail if taps > 1 else None), _ptr(out), _ptr(out_bf16), n, _stream()),
        f"ssm_conv ({c} channels, {taps} taps)", n_kernels=2 if taps > 1 else 1)


def ssm_scan(xbc, proj, dt_off: int, dt_bias, a_log, d_skip, cu_q, seq_slot, n_seqs: int, heads: int, groups: int, n_state: int,
             vdim: int, state, y, chunked: bool = False) -> None:
    """The recurrence ``S_t = exp(-exp(a_log) dt_t) S_(t-1) + dt_t B_t x_t^T``, ``y_t = S_t^T C_t + D x_t`` per head, with
    ``dt_t = softplus(proj[t, dt_off + head] + dt_bias)``; ``xbc [n, heads*vdim + 2*groups*n_state]`` holds x, B, C after
    the convolution; ``state [slots, heads, n_state, vdim]`` float32 is read and left advanced; ``y [n, heads*vdim]``."""
    n, ch = xbc.shape
    inner = heads * vdim
    _need(xbc, "xbc", torch.float32, (n, inner + 2 * groups * n_state))
    _need(proj, "proj", torch.float32, (n, None))
    for t, nm in ((dt_bias, "dt_bias"), (a_log, "a_log"), (d_skip, "d_skip")):
        _need(t, nm, torch.float32, (heads,))
    _need(state, "state", torch.float32, (None, heads, n_state, vdim))
    _need(y, "y", torch.float32, (n, inner))
    for t, nm in ((cu_q, "cu_q"), (seq_slot, "seq_slot")):
        _need(t, nm, torch.int32)
    if dt_off < 0 or dt_off + heads > proj.shape[1]:
        raise KernelError(f"ssm_scan: {heads} step sizes from column {dt_off} of a row of {proj.shape[1]}")
    if chunked:
        # a step of many tokens: chunks side by side (own states from zero, a prefix over them, outputs from the start states)
        cht = max(SSM_CHUNK_TOKENS, -(-n // 64 // 32) * 32)
        n_chunks = n // cht + int(n_seqs)
        cstate = torch.empty((n_chunks, heads, n_state, vdim), dtype=torch.float32, device=xbc.device)
        cdec = torch.empty((n_chunks, heads), dtype=torch.float32, device=xbc.device)
        _ok(ssm_lib().dryft_ssm_scan_chunked(_ptr(xbc), ch, _ptr(proj), proj.shape[1], int(dt_off), _ptr(dt_bias), _ptr(a_log),
                                             _ptr(d_skip), _ptr(cu_q), _ptr(seq_slot), int(n_seqs), cht, n_chunks, heads, groups,
                                             n_state, vdim, _ptr(state), _ptr(cstate), _ptr(cdec), _ptr(y), _stream()),
            f"ssm_scan_chunked ({heads} heads, state {n_state} x {vdim})", n_kernels=3)
        return
    _ok(ssm_lib().dryft_ssm_scan(_ptr(xbc), ch, _ptr(proj), proj.shape[1], int(dt_off), _ptr(dt_bias), _ptr(a_log), _ptr(d_skip),
                                 _ptr(cu_q), _ptr(seq_slot), int(n_seqs), heads, groups, n_state, vdim, _ptr(state), _ptr(y),
                                 _stream()), f"ssm_scan ({heads} heads, state {n_state} x {vdim})")


# ----------------------------------------------------------------------------- windowed attention with pooled blocks and a sink
def pool_attention_lib(qk_dim: int, v_dim: int, group: int) -> ctypes.CDLL:
    if qk_dim <= 0 or v_dim <= 0 or qk_dim > 512 or v_dim > 512:
        raise KernelError(f"pooled-window attention takes key and value sizes up to 512, got {qk_dim}, {v_dim}")
    if group < 1 or group > 16:
        raise KernelError(f"pooled-window attention takes 1..16 query heads per kv head, got {group}")
    key = ("pool_attn", qk_dim, v_dim, group)
    with _lock:
        lib = _variants.get(key)
        if lib is None:
            path = build.build_library("pool_attn", ("pool_attn.cu",),
                                       {"DRYFT_QK_DIM": qk_dim, "DRYFT_V_DIM": v_dim, "DRYFT_GROUP": group})
            lib = _load(path)
            lib.dryft_pool_attn_prep.argtypes = [_i, _p, _i, _p, _p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _f,
                                                 _i, _p]
            lib.dryft_pool_attn_blocks.argtypes = [_i, _p, _p, _p, _i, _i, _p, _p, _p, _i, _p, _p, _i, _i, _i, _p]
            lib.dryft_pool_attn_rows.argtypes = [_i, _p, _p, _p, _p, _i, _i, _p, _p, _p, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _f,
                                                 _i, _i, _p]
            lib.dryft_pool_attn_prep_tok.argtypes = [_i, _p, _i, _p, _p, _f, _p, _p, _i, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i,
                                                     _f, _i, _p]
            for fn in ("dryft_pool_attn_prep", "dryft_pool_attn_prep_tok", "dryft_pool_attn_blocks", "dryft_pool_attn_rows"):
                getattr(lib, fn).restype = _i
            if (lib.dryft_pool_attn_qk_dim(), lib.dryft_pool_attn_v_dim(), lib.dryft_pool_attn_group()) != (qk_dim, v_dim, group):
                raise KernelError(f"{path} was compiled for other sizes")
            _variants[key] = lib
        return lib


def pool_attention_prefill_supported(qk_dim: int, v_dim: int, group: int, page: int = 64) -> bool:
    """Whether the tensor-core prompt kernel of the pooled-window attention takes this head shape (k16 steps over the keys,
    n8 pairs over the values, 64-token pages, two stages of a key and a value tile in shared memory)."""
    return (qk_dim > 0 and qk_dim % 16 == 0 and qk_dim <= 256 and v_dim > 0 and v_dim % 16 == 0 and v_dim <= 256
            and page == 64 and 1 <= group <= 16 and 2 * ((64 + 128) * (qk_dim + 8) + 128 * (v_dim + 8)) <= 227 * 1024)


def pool_attention_prefill_lib(qk_dim: int, v_dim: int, group: int, page: int = 64) -> ctypes.CDLL:
    if not pool_attention_prefill_supported(qk_dim, v_dim, group, page):
        raise KernelError(f"pooled-window prompt attention takes key and value sizes in steps of 16 and 64-token pages, got "
                          f"{qk_dim}, {v_dim}, {page}")
    key = ("pool_prefill", qk_dim, v_dim, group, page)
    with _lock:
        lib = _variants.get(key)
        if lib is None:
            path = build.build_library("pool_attn_prefill", ("pool_attn_prefill.cu",),
                                       {"DRYFT_QK_DIM": qk_dim, "DRYFT_V_DIM": v_dim, "DRYFT_GROUP": group, "DRYFT_PAGE": page})
            lib = _load(path)
            lib.dryft_pool_attn_prefill.argtypes = [_p, _p, _p, _p, _i, _i, _p, _p, _p, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _f,
                                                    _i, _i, _p]
            lib.dryft_pool_attn_prefill.restype = _i
            if (lib.dryft_pool_attn_prefill_qk_dim(), lib.dryft_pool_attn_prefill_v_dim()) != (qk_dim, v_dim):
                raise KernelError("pooled-window prompt attention: the library was built for another head shape")
            _variants[key] = lib
        return lib


def pool_attn_prefill(q, k_pages, v_pages, page_table, pooled, sink, tile_tok0, tile_rows, tok_slot, tok_pos, out, n_tiles: int,
                      scale: float, size: int, pool: int) -> None:
    """Prompt attention (bfloat16) of ``q [n, H, D]``, tile by tile of up to 64 tokens of one sequence, over the last ``size``
    cached tokens and the pooled rows of the blocks of ``pool`` positions wholly before them (``pooled = (pk_pages, pv_pages,
    pool_table)``; ``pool = 0``: none); the softmax's denominator also holds ``exp(sink[head])`` (if given)."""
    n, n_heads, d = q.shape
    n_kv, page = k_pages.shape[1], k_pages.shape[2]
    dv = v_pages.shape[-1]
    _need(q, "q", torch.bfloat16)
    _need(k_pages, "k_pages", q.dtype, (None, n_kv, page, d))
    _need(v_pages, "v_pages", q.dtype, (None, n_kv, page, dv))
    _need(out, "out", q.dtype, (n, n_heads, dv))
    _need(page_table, "page_table", torch.int32)
    if sink is not None:
        _need(sink, "sink", torch.float32, (n_heads,))
    pk = pv = pt = None
    if pool:
        pk, pv, pt = pooled
        _need(pk, "pk_pages", q.dtype, (None, n_kv, page, d))
        _need(pv, "pv_pages", q.dtype, (None, n_kv, page, dv))
        _need(pt, "pool_table", torch.int32)
    lib = pool_attention_prefill_lib(d, dv, n_heads // n_kv, page)
    _ok(lib.dryft_pool_attn_prefill(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1], page, _ptr(pk),
                                    _ptr(pv), _ptr(pt), pt.shape[1] if pt is not None else 0, _ptr(sink), _ptr(tile_tok0),
                                    _ptr(tile_rows), _ptr(tok_slot), _ptr(tok_pos), _ptr(out), int(n_tiles), n_heads, n_kv,
                                    float(scale), int(size), int(pool), _stream()),
        f"pool_attn_prefill (window {size}, blocks of {pool})")


def pool_attn_prep(proj, q_bias, k_bias, v_bias, inv_freq, inv_freq_lo, rot: int, tok_slot, tok_pos, q_out, k_pages, v_pages,
                   page_table, n_heads: int, n_kv: int, eps: float, write_kv: bool) -> None:
    """Per token of ``proj [n, H*D (+ G*D + G*DV)]``: bias, rotation of the first ``rot`` dims (rotate-half), division by the
    root mean square over the head (no weight; ``eps < 0``: not divided) for q and k; v plus its bias; k and v into the cache
    pages."""
    n, ld = proj.shape
    d, dv = q_out.shape[2], v_pages.shape[-1]
    _need(proj, "proj")
    _need(q_out, "q_out", proj.dtype, (n, n_heads, d))
    _need(k_pages, "k_pages", proj.dtype, (None, n_kv, None, d))
    _need(v_pages, "v_pages", proj.dtype, (None, n_kv, k_pages.shape[2], dv))
    _need(page_table, "page_table", torch.int32)
    if ld < n_heads * d + (n_kv * (d + dv) if write_kv else 0):
        raise KernelError(f"pool_attn_prep: a row of {ld} values is too short for {n_heads} + {n_kv} heads")
    for t, nm, cnt in ((q_bias, "q_bias", n_heads * d), (k_bias, "k_bias", n_kv * d), (v_bias, "v_bias", n_kv * dv)):
        if t is not None:
            _need(t, nm, torch.float32, (cnt,))
    if rot:
        _need(inv_freq, "inv_freq", torch.float32, (rot // 2,))
        if inv_freq_lo is not None:
            _need(inv_freq_lo, "inv_freq_lo", torch.float32, (rot // 2,))
    lib = pool_attention_lib(d, dv, n_heads // n_kv)
    _ok(lib.dryft_pool_attn_prep(_act(proj, "proj"), _ptr(proj), ld, _ptr(q_bias), _ptr(k_bias), _ptr(v_bias), _ptr(inv_freq),
                                 _ptr(inv_freq_lo), int(rot), _ptr(tok_slot), _ptr(tok_pos), _ptr(q_out), _ptr(k_pages), _ptr(v_pages),
                                 _ptr(page_table), page_table.shape[1], k_pages.shape[2], n, n_heads, n_kv, float(eps),
                                 int(write_kv), _stream()), f"pool_attn_prep ({n_heads}/{n_kv} heads of {d})")


def pool_attn_prep_tok(proj, q_norm_w, k_norm_w, norm_eps: float, inv_freq, inv_freq_lo, rot: int, interleaved: bool, tok_slot, tok_pos,
                       q_out, k_pages, v_pages, page_table, n_heads: int, n_kv: int, eps: float, write_kv: bool) -> None:
    """``pool_attn_prep`` for projections normed as a whole: per token of ``proj [n, H*D (+ G*D + G*DV)]`` all of q (and all of k)
    is divided by its root mean square (``norm_eps`` inside the root) and multiplied by ``q_norm_w [H*D]`` (``k_norm_w [G*D]``)
    BEFORE the rotation of each head's first ``rot`` dims (``interleaved``: dims ``2i`` and ``2i + 1`` turn together, else
    ``i`` and ``i + rot/2``); then the optional unit norm per head (``eps >= 0``); k and v into the cache pages."""
    n, ld = proj.shape
    d, dv = q_out.shape[2], v_pages.shape[-1]
    _need(proj, "proj")
    _need(q_out, "q_out", proj.dtype, (n, n_heads, d))
    _need(k_pages, "k_pages", proj.dtype, (None, n_kv, None, d))
    _need(v_pages, "v_pages", proj.dtype, (None, n_kv, k_pages.shape[2], dv))
    _need(page_table, "page_table", torch.int32)
    if ld < n_heads * d + (n_kv * (d + dv) if write_kv else 0):
        raise KernelError(f"pool_attn_prep_tok: a row of {ld} values is too short for {n_heads} + {n_kv} heads")
    if q_norm_w is not None:
        _need(q_norm_w, "q_norm_w", torch.float32, (n_heads * d,))
    if k_norm_w is not None:
        _need(k_norm_w, "k_norm_w", torch.float32, (n_kv * d,))
    if rot:
        _need(inv_freq, "inv_freq", torch.float32, (rot // 2,))
        if inv_freq_lo is not None:
            _need(inv_freq_lo, "inv_freq_lo", torch.float32, (rot // 2,))
    lib = pool_attention_lib(d, dv, n_heads // n_kv)
    _ok(lib.dryft_pool_attn_prep_tok(_act(proj, "proj"), _ptr(proj), ld, _ptr(q_norm_w), _ptr(k_norm_w), float(norm_eps), _ptr(inv_freq),
                                     _ptr(inv_freq_lo), int(rot), int(interleaved), _ptr(tok_slot), _ptr(tok_pos), _ptr(q_out),
                                     _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1], k_pages.shape[2], n, n_heads,
                                     n_kv, float(eps), int(write_kv), _stream()), f"pool_attn_prep_tok ({n_heads}/{n_kv} heads of {d})")


def pool_attn_blocks(k_pages, v_pages, page_table, pk_pages, pv_pages, pool_table, tok_slot, tok_pos, n: int, pool: int,
                     group: int) -> None:
    """Every token of the step that completes a block of ``pool`` positions leaves the means of the block's cached keys and
    values in the pooled pages."""
    n_kv, page, d = k_pages.shape[1], k_pages.shape[2], k_pages.shape[3]
    dv = v_pages.shape[-1]
    _need(k_pages, "k_pages")
    _need(v_pages, "v_pages", k_pages.dtype)
    _need(pk_pages, "pk_pages", k_pages.dtype, (None, n_kv, page, d))
    _need(pv_pages, "pv_pages", k_pages.dtype, (None, n_kv, page, dv))
    _need(pool_table, "pool_table", torch.int32)
    lib = pool_attention_lib(d, dv, group)
    _ok(lib.dryft_pool_attn_blocks(_act(k_pages, "k_pages"), _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1], page,
                                   _ptr(pk_pages), _ptr(pv_pages), _ptr(pool_table), pool_table.shape[1], _ptr(tok_slot), _ptr(tok_pos),
                                   n, n_kv, int(pool), _stream()), f"pool_attn_blocks (blocks of {pool})")


def pool_attn_rows(q, k_pages, v_pages, page_table, pooled, sink, tok_slot, tok_pos, out, scale: float, size: int, pool: int,
                   n_splits: int = 1, part_o=None, part_ml=None) -> None:
    """Row-wise attention of ``q [n, H, D]`` over the last ``size`` cached tokens and, beside them, the pooled row of every block
    of ``pool`` positions that lies wholly before them (``pooled = (pk_pages, pv_pages, pool_table)``; ``pool = 0``: none), one
    softmax whose denominator also holds ``exp(sink[head])`` (if given).  ``out [n, H, DV]``."""
    n, n_heads, d = q.shape
    n_kv, page = k_pages.shape[1], k_pages.shape[2]
    dv = v_pages.shape[-1]
    _need(q, "q")
    _need(k_pages, "k_pages", q.dtype, (None, n_kv, page, d))
    _need(v_pages, "v_pages", q.dtype, (None, n_kv, page, dv))
    _need(out, "out", q.dtype, (n, n_heads, dv))
    if sink is not None:
        _need(sink, "sink", torch.float32, (n_heads,))
    pk = pv = pt = None
    if pool:
        pk, pv, pt = pooled
        _need(pk, "pk_pages", q.dtype, (None, n_kv, page, d))
        _need(pv, "pv_pages", q.dtype, (None, n_kv, page, dv))
        _need(pt, "pool_table", torch.int32)
    if n_splits > 1:
        _need(part_o, "part_o", torch.float32, (n, n_heads, n_splits, dv))
        _need(part_ml, "part_ml", torch.float32, (n, n_heads, n_splits, 2))
    lib = pool_attention_lib(d, dv, n_heads // n_kv)
    _ok(lib.dryft_pool_attn_rows(_act(q, "q"), _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1], page,
                                 _ptr(pk), _ptr(pv), _ptr(pt), pt.shape[1] if pt is not None else 0, _ptr(sink), _ptr(tok_slot),
                                 _ptr(tok_pos), _ptr(out), _ptr(part_o), _ptr(part_ml), n, n_kv, int(n_splits), float(scale), int(size),
                                 int(pool), _stream()), f"pool_attn_rows (window {size}, blocks of {pool})",
        n_kernels=2 if n_splits > 1 else 1)


# ----------------------------------------------------------------------------- a 32-bit stream that takes several results at once
def stream_par_lib() -> ctypes.CDLL:
    return _single_lib("stream_par", {
        "dryft_stream_sum": [_i, _p, _p, _p, _f, _p, _f, _p, _f, _p, _i, _f, _p, _p, _f, _p, _i, _i, _p],
        "dryft_pack_pair": [_i, _p, _p, _p, _i, _i, _p],
        "dryft_softcap": [_p, _ll, _f, _p],
    })


def stream_sum(x32, terms=(), *, rows=None, top: int = 0, rows_scale: float = 1.0, vec=None, src=None, norm_w=None, eps: float = 0.0,
               h=None) -> None:
    """``x32[n] (or src[n]) + sum_i scale_i * y_i[n] + rows_scale * sum_k rows[n * top + k] + vec -> x32[n]`` in 32-bit, for up
    to three ``terms`` ``(y_i, scale_i)`` of the activation type ``[n, width]``, ``rows [n * top, width]`` (a routed
    feed-forward's results, summed in the order of the choices) and a 32-bit vector ``vec [width]``; with ``norm_w`` also
    ``h[n] = T(x32[n] / sqrt(mean(x32[n]^2) + eps) * norm_w)``, the next layer's normed input."""
    n, width = x32.shape
    _need(x32, "x32", torch.float32)
    terms = [(y, float(sc)) for y, sc in terms if y is not None]
    if len(terms) > 3:
        raise KernelError("stream_sum: at most three terms beside the routed rows")
    act = None
    for y, _ in terms:
        _need(y, "term", act, (n, width))
        act = y.dtype
    if rows is not None:
        if top < 1:
            raise KernelError("stream_sum: routed rows need their count per token")
        _need(rows, "rows", act, (n * top, width))
        act = rows.dtype
    if h is not None:
        _need(h, "h", act, (n, width))
        act = h.dtype
    if src is not None:
        _need(src, "src", torch.float32, (n, width))
    if vec is not None:
        _need(vec, "vec", torch.float32, (width,))
    if norm_w is not None:
        _need(norm_w, "norm_w", torch.float32, (width,))
        if h is None:
            raise KernelError("stream_sum: a norm needs the tensor its result goes to")
    if act is None:
        act = torch.float32
    if act not in (torch.float32, torch.bfloat16):
        raise KernelError(f"stream_sum: terms are float32 or bfloat16, got {act}")
    terms += [(None, 0.0)] * (3 - len(terms))
    _ok(stream_par_lib().dryft_stream_sum(int(act == torch.bfloat16), _ptr(x32), _ptr(src), _ptr(terms[0][0]), terms[0][1],
                                          _ptr(terms[1][0]), terms[1][1], _ptr(terms[2][0]), terms[2][1], _ptr(rows), int(top),
                                          float(rows_scale), _ptr(vec), _ptr(norm_w), float(eps), _ptr(h if norm_w is not None else None),
                                          n, width, _stream()), "stream_sum")


def pack_pair(a32, b32, out) -> None:
    """``out[n] = T([a32[n] | b32[n]])``: two 32-bit rows side by side as one operand row."""
    n, width = a32.shape
    _need(a32, "a32", torch.float32)
    _need(b32, "b32", torch.float32, (n, width))
    _need(out, "out", None, (n, 2 * width))
    _ok(stream_par_lib().dryft_pack_pair(_act(out, "out"), _ptr(a32), _ptr(b32), _ptr(out), n, width, _stream()), "pack_pair")


def softcap(logits, cap: float) -> None:
    """``logits <- cap * tanh(logits / cap)`` in place (float32)."""
    _need(logits, "logits", torch.float32)
    _ok(stream_par_lib().dryft_softcap(_ptr(logits), logits.numel(), float(cap), _stream()), "softcap")


# ----------------------------------------------------------------------------- selective scan (a decay per channel and state)
SELSCAN_MAX_STATE = 512
SELSCAN_CHUNK_TOKENS = 64


def selscan_lib() -> ctypes.CDLL:
    return _single_lib("selscan", {
        "dryft_selscan": [_i, _p, _p, _i, _i, _i, _p, _p, _p, _p, _p, _i, _i, _p, _p, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p],
    })


def selscan(xc, low, b_off: int, c_off: int, dtp, dt_bias, a_log, d_skip, zrows, z_off: int, cu_q, seq_slot, n_seqs: int, state, out,
            chunked: bool = False) -> None:
    """``S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x[t, c] B[t, n]``, ``y[t, c] = sum_n S[c, n] C[t, n] + D[c] x[t, c]``,
    ``out[t, c] = T(y * silu(z[t, c]))`` with ``dt_c = softplus(dtp[t, c] + dt_bias[c])`` and ``A = -exp(a_log)``: ``xc [n,
    inner]``, ``dtp [n, inner]`` float32; B and C are ``N`` columns of ``low [n, ld]`` (float32) from ``b_off`` / ``c_off``; z
    ``inner`` columns of ``zrows [n, ld']`` (float32) from ``z_off``; ``state [slots, inner, N]`` float32 is read and left
    advanced.  ``chunked``: a step of many tokens runs its chunks side by side (three launches)."""
    n, inner = xc.shape
    n_state = a_log.shape[1]
    _need(xc, "xc", torch.float32)
    _need(dtp, "dtp", torch.float32, (n, inner))
    _need(low, "low", torch.float32, (n, None))
    _need(zrows, "zrows", torch.float32, (n, None))
    _need(a_log, "a_log", torch.float32, (inner, n_state))
    for t, nm in ((dt_bias, "dt_bias"), (d_skip, "d_skip")):
        _need(t, nm, torch.float32, (inner,))
    _need(state, "state", torch.float32, (None, inner, n_state))
    _need(out, "out", None, (n, inner))
    for t, nm in ((cu_q, "cu_q"), (seq_slot, "seq_slot")):
        _need(t, nm, torch.int32)
    if min(b_off, c_off) < 0 or max(b_off, c_off) + n_state > low.shape[1] or z_off < 0 or z_off + inner > zrows.shape[1]:
        raise KernelError("selscan: B, C or z columns outside their rows")
    cht = n_chunks = 0
    cstate = cdt = None
    if chunked:
        cht = max(SELSCAN_CHUNK_TOKENS, -(-n // 64 // 32) * 32)
        n_chunks = n // cht + int(n_seqs)
        cstate = torch.empty((n_chunks, inner, n_state), dtype=torch.float32, device=xc.device)
        cdt = torch.empty((n_chunks, inner), dtype=torch.float32, device=xc.device)
    _ok(selscan_lib().dryft_selscan(_act(out, "out"), _ptr(xc), _ptr(low), low.shape[1], int(b_off), int(c_off), _ptr(dtp), _ptr(dt_bias),
                                    _ptr(a_log), _ptr(d_skip), _ptr(zrows), zrows.shape[1], int(z_off), _ptr(cu_q), _ptr(seq_slot),
                                    int(n_seqs), cht, n_chunks, inner, n_state, _ptr(state), _ptr(cstate), _ptr(cdt), _ptr(out), _stream()),
        f"selscan ({inner} channels, state {n_state})", n_kernels=3 if chunked else 1)
