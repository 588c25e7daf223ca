"""Python faces of the CUDA kernels.

Each function checks shapes and dtypes, then calls one launcher of the kernel
library through its C symbol on torch's current stream.  Nothing here computes:
there is no CPU or library fallback, and a missing or unloadable library is an
error at first use.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build as _build

ACT_NONE, ACT_GELU_TANH, ACT_GELU_ERF = 0, 1, 2
ACT_CODES = {None: ACT_NONE, "none": ACT_NONE, "tanh": ACT_GELU_TANH, "erf": ACT_GELU_ERF}

STATUS_OK, STATUS_BAD_PAGE, STATUS_WAIT_TIMEOUT = 0, 1, 2
_ERR_NAMES = {-1: "bad argument", -2: "unsupported size", -3: "CUDA driver call failed"}


class KernelError(RuntimeError):
    pass


_lib = None

_c_int, _c_float, _c_ptr = ctypes.c_int, ctypes.c_float, ctypes.c_void_p

_SIGNATURES = {
    "nib_embed": [_c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr],
    "nib_layernorm": [_c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_float, _c_ptr],
    "nib_kv_append": [_c_int, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr,
                      _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "nib_linear_simt": [_c_int, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int,
                        _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr],
    "nib_linear_tc_supported": [_c_ptr, _c_int, _c_ptr, _c_int, _c_int],
    "nib_linear_tc": [_c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                      _c_int, _c_int, _c_ptr, _c_ptr],
    "nib_linear_tc_small": [_c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                            _c_int, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_ptr, _c_ptr,
                            _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr,
                            ctypes.c_longlong, _c_ptr, _c_int, _c_ptr, _c_ptr],
    "nib_linear_tc_pair_supported": [_c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int],
    "nib_linear_tc_pair": [_c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                           _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                           _c_int, _c_int, _c_ptr, _c_ptr],
    "nib_linear_skinny_supported": [_c_int, _c_int, _c_int, _c_int, _c_ptr],
    "nib_linear_skinny": [_c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                          _c_int, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_ptr, _c_ptr,
                          _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "nib_attention_prefill_tc_supported": [_c_int, _c_int],
    "nib_attention_prefill_tc": [_c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr,
                                 _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_ptr, _c_ptr],
    "nib_attention_simt": [_c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr,
                           _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_ptr, _c_ptr],
    "nib_attention_decode": [_c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr,
                             _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int,
                             _c_int, _c_ptr, _c_ptr, _c_ptr],
    "nib_attention_decode_mma_supported": [_c_int, _c_int],
    "nib_attention_decode_mma_clusters": [_c_int, _c_int],
    "nib_attention_decode_mma": [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr,
                                 _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int,
                                 _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr],
    "nib_attention_prefill_supported": [_c_int],
    "nib_attention_prefill": [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr,
                              _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_ptr, _c_ptr],
    "nib_convert": [_c_int, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, ctypes.c_longlong, ctypes.c_longlong, _c_int, _c_ptr],
    "nib_argmax": [_c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "nib_sample": [_c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int,
                   _c_ptr],
}


#: the active trace recorder (``trace.start`` puts it here), or None
_rec = None


def _recorder():
    return _rec


#: the analytic description of the launch about to be made (set by the faces while a recorder is active)
_pending_op = None


def _note(kind: str, name: str, dims, flops: float, nbytes: float) -> None:
    global _pending_op
    from ..trace import Op
    _pending_op = Op(kind, name, tuple(int(d) for d in dims), float(flops), float(nbytes))


def tracing() -> bool:
    """Whether a trace recorder is active (the faces then describe every launch to it)."""
    return _rec is not None


def trace_scope(layer: int = -1, name: str = "") -> None:
    """Tell the active recorder which layer, and which named product, the next launches belong to."""
    if _rec is not None:
        _rec.layer, _rec.name = layer, name


class _Library:
    """The launchers of the kernel library; with a trace recorder active each call is bracketed by events."""

    def __init__(self, lib: ctypes.CDLL):
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _c_int
            setattr(self, name, self._wrap(name, fn))
        self.raw = lib

    @staticmethod
    def _wrap(name, fn):
        counted = name not in ("nib_linear_tc_supported", "nib_linear_tc_pair_supported", "nib_linear_skinny_supported",
                               "nib_attention_prefill_tc_supported", "nib_attention_prefill_supported",
                               "nib_attention_decode_mma_supported", "nib_attention_decode_mma_clusters")

        def call(*args):
            global _pending_op
            rec = _recorder() if counted else None
            if rec is None:
                return fn(*args)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            code = fn(*args)
            e1.record()
            op, _pending_op = _pending_op, None
            if code == 0:
                if op is None:
                    from ..trace import Op
                    op = Op("other", name[4:], (0, 0, 0), 0.0, 0.0)
                rec.add(op, name, e0, e1)
            return code
        return call


def library() -> _Library:
    """The loaded kernel library; compiled on first use if the built file is missing."""
    global _lib
    if _lib is None:
        if not torch.cuda.is_available():
            raise KernelError("nanoinfer_b200 needs a CUDA device: there is no CPU path")
        path = _build.library_path(build=True)
        _lib = _Library(ctypes.CDLL(path))
    return _lib


_bound_stream: Optional[int] = None


def _stream() -> int:
    """The stream that kernels are enqueued on: torch's current stream, looked up once per step when
    the step function has bound it (the look-up costs more than a launch does)."""
    return _bound_stream if _bound_stream is not None else torch.cuda.current_stream().cuda_stream


class bound_stream:
    """``with bound_stream():`` every launch inside goes to the stream that is current on entry."""

    def __enter__(self):
        global _bound_stream
        self._before = _bound_stream
        _bound_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _bound_stream
        _bound_stream = self._before
        return False


_launches = 0


def launch_count() -> int:
    """How many kernels this process has enqueued through this interface (captured launches count once)."""
    return _launches


def _check(code: int, what: str, kernels: int = 1) -> None:
    global _launches
    if code == 0:
        _launches += kernels
        return
    if code < 0:
        raise KernelError(f"{what}: {_ERR_NAMES.get(code, code)}")
    raise KernelError(f"{what}: CUDA error {code}")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"dtype {t.dtype} is not supported by the kernels")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _i32(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")


# ------------------------------------------------------------------------------ ops
def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
          pos_table: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None,
          feedback: Optional[torch.Tensor] = None) -> None:
    """out[t] = table[tokens[t]] (+ pos_table[positions[t]]), written as 32-bit floats.  A negative
    token -(s + 1) stands for ``feedback[s]``, the token that the step before left on the device for
    slot s."""
    T, C = tokens.shape[0], table.shape[1]
    _i32(tokens, "tokens")
    if out.dtype != torch.float32 or out.shape[0] < T or out.shape[1] != C or not out.is_contiguous():
        raise KernelError("embed: out must be contiguous float32 [T, C]")
    if pos_table is not None:
        if positions is None or pos_table.dtype != table.dtype or pos_table.shape[1] != C:
            raise KernelError("embed: pos_table needs positions, the table's dtype and its width")
        _i32(positions, "positions")
    if feedback is not None:
        _i32(feedback, "feedback")
    if tracing():
        _note("embed", "embed", (T, C, 0), T * C, T * C * ((2 if pos_table is not None else 1) * table.element_size() + 4))
    _check(library().nib_embed(_dt(table), _ptr(tokens), _ptr(positions), _ptr(table), _ptr(pos_table),
                               _ptr(feedback), _ptr(out), T, C, _stream()), "embed")


def layernorm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float, out: torch.Tensor,
              n_rows: int, rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = LayerNorm(x[rows[r]] if rows is given else x[r]); x is the 32-bit residual stream."""
    C = x.shape[1]
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("layernorm: x must be contiguous float32")
    if gamma.dtype != torch.float32 or beta.dtype != torch.float32 or gamma.numel() != C or beta.numel() != C:
        raise KernelError("layernorm: gamma and beta must be float32 [C]")
    if out.shape[1] != C or out.shape[0] < n_rows or not out.is_contiguous():
        raise KernelError("layernorm: out must be contiguous [n_rows, C]")
    if rows is not None:
        _i32(rows, "rows")
    if tracing():
        _note("ln", "ln", (n_rows, C, 0), 8.0 * n_rows * C, n_rows * C * (4 + out.element_size()) + 8 * C)
    _check(library().nib_layernorm(_dt(out), _ptr(x), _ptr(rows), _ptr(gamma), _ptr(beta), _ptr(out),
                                   n_rows, C, float(eps), _stream()), "layernorm")


def linear_simt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, M: int,
                act: int = ACT_NONE, residual: bool = False) -> None:
    """out[:M] = act(a[:M] . w^T + bias) on the CUDA cores; with residual, added to the 32-bit out."""
    N, K = w.shape
    if a.shape[1] != K or a.dtype != w.dtype or a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("linear: a [M, K] and w [N, K] must share K and dtype, rows contiguous")
    if out.shape[1] != N or out.shape[0] < M or a.shape[0] < M:
        raise KernelError("linear: out must be [M, N]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("linear: bias must be float32 [N]")
    _check(library().nib_linear_simt(_dt(a), _dt(out), _ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(bias),
                                     _ptr(out), out.stride(0), M, N, K, act, int(residual), _stream()),
           "linear_simt")


_status: Optional[torch.Tensor] = None


def status_word() -> torch.Tensor:
    """The device status word (int32 [1]) that kernels write when they meet a fault they can
    name (a page index outside its pool, a wait that ran out).  0 means fine."""
    global _status
    if _status is None:
        _status = torch.zeros(1, dtype=torch.int32, device="cuda")
    return _status


def linear_tc(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, M: int,
              act: int = ACT_NONE, residual: bool = False) -> None:
    """out[:M] = act(a[:M] . w^T + bias) for bfloat16 a and w on the tensor cores (tcgen05, TMA)."""
    N, K = w.shape
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.shape[1] != K:
        raise KernelError("linear_tc: a [M, K] and w [N, K] must be bfloat16 and share K")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1 or out.shape[1] != N or out.shape[0] < M:
        raise KernelError("linear_tc: rows must be contiguous and out [M, N]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("linear_tc: bias must be float32 [N]")
    _check(library().nib_linear_tc(_dt(out), _ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out),
                                   out.stride(0), M, N, K, act, int(residual), _ptr(status_word()), _stream()),
           "linear_tc")


_capability: dict = {}


def _can(name: str, *args) -> bool:
    """A capability query of the library, remembered: the answers depend on sizes and alignments
    only, and a foreign-function call costs about as much as a launch."""
    key = (name,) + args
    got = _capability.get(key)
    if got is None:
        got = _capability[key] = bool(getattr(library(), name)(*args))
    return got


def linear_tc_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    return bool(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.stride(1) == 1 and w.stride(1) == 1
                and _can("nib_linear_tc_supported", 16 + (_ptr(a) & 15), a.stride(0), 16 + (_ptr(w) & 15), w.stride(0),
                         w.shape[1]))   # (only the alignment of the pointers matters: 16 + the low bits)


def linear_tc_pair(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, M: int,
                   act: int = ACT_NONE, residual: bool = False, bq: int = 0, splits: int = 0, kv=None) -> bool:
    """The tcgen05 product for many rows by pairs of blocks (one 256-row MMA over two SMs, each block
    loading half of the weight tile).  ``kv``: (cache layer, block table, row_entry, positions, q_dim)
    sends keys and values straight to the cache.  False if the shape or an alignment is not taken."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.stride(1) != 1 or w.stride(1) != 1 \
            or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
        return False
    N, K = w.shape
    if not _can("nib_linear_tc_pair_supported", _dt(out), 16 + (_ptr(a) & 15), a.stride(0), 16 + (_ptr(w) & 15),
                w.stride(0), 16 + (_ptr(out) & 15), out.stride(0), M, N, K, int(residual)):
        return False
    _, kv_args = _option_args(None, kv)
    if kv is not None and (kv[4] % 64 or kv[0].shape[4] % 16 or out.dtype != torch.bfloat16 or residual):
        return False
    if tracing():
        _note_linear(a, None, w, bias, out, M, residual)
    _check(library().nib_linear_tc_pair(_dt(out), _ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out),
                                        out.stride(0), M, N, K, act, int(residual), int(bq), int(splits), *kv_args,
                                        _ptr(status_word()), _stream()), "linear_tc_pair")
    return True


def _note_linear(a, norm, w, bias, out, M, residual) -> None:
    """[M, K, N]: 2 M K N + M N FLOPs; weights, bias, input and output once (the residual stream is read
    and written where the product adds into it)."""
    N, K = w.shape
    in_bytes = M * K * (4 if norm is not None else a.element_size())
    out_bytes = M * N * out.element_size() * (2 if residual else 1)
    _note("matmul", "matmul", (M, K, N), 2.0 * M * K * N + M * N,
          N * K * w.element_size() + (4 * N if bias is not None else 0) + in_bytes + out_bytes)


class NormInput:
    """Activations given as the 32-bit residual stream plus the parameters of the LayerNorm that
    stands before the product: ``linear`` normalises ``x[rows[m]]`` (or ``x[m]``) itself, inside the
    tensor-core kernel where the step is small enough, else with the LayerNorm kernel into scratch
    taken from ``workspace``."""

    def __init__(self, x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float, workspace,
                 dtype: torch.dtype, rows: Optional[torch.Tensor] = None, max_rows: int = 0):
        self.x, self.gamma, self.beta, self.eps = x, gamma, beta, float(eps)
        self.workspace, self.dtype, self.rows, self.max_rows = workspace, dtype, rows, max_rows

    def materialise(self, M: int) -> torch.Tensor:
        out = self.workspace.get("norm.fallback", (max(M, self.max_rows), self.x.shape[1]), self.dtype)
        layernorm(self.x, self.gamma, self.beta, self.eps, out, M, self.rows)
        return out


SMALL_STEP_MAX_ROWS = 128
_split_scratch: Optional[torch.Tensor] = None
_split_counters: Optional[torch.Tensor] = None


def _split_buffers(device):
    """Scratch for the K splits of small steps: 4 M floats of partial tiles and 4096 tile counters
    (found zero and left zero by the kernel), allocated once."""
    global _split_scratch, _split_counters
    if _split_scratch is None:
        _split_scratch = torch.empty(4 << 20, dtype=torch.float32, device=device)
        _split_counters = torch.zeros(4096, dtype=torch.int32, device=device)
    return _split_scratch, _split_counters


def _option_args(norm, kv):
    if kv is not None:
        cache, block_table, row_entry, positions, q_dim = kv
        n_pages, _, n_kv_head, page_size, head_dim = cache.shape
        kv_args = (_ptr(cache), _ptr(block_table), block_table.shape[1], _ptr(row_entry), _ptr(positions), q_dim,
                   n_kv_head, head_dim, page_size, n_pages)
    else:
        kv_args = (None, None, 0, None, None, 0, 0, 0, 0, 0)
    if norm is not None:
        ln_args = (_ptr(norm.x), norm.x.stride(0), _ptr(norm.gamma), _ptr(norm.beta), norm.eps, _ptr(norm.rows))
    else:
        ln_args = (None, 0, None, None, 0.0, None)
    return ln_args, kv_args


def _small_inputs_ok(a, norm, w, out) -> bool:
    if w.dtype != torch.bfloat16 or w.stride(1) != 1 or out.stride(1) != 1:
        return False
    if a is not None and (a.dtype != torch.bfloat16 or a.stride(1) != 1):
        return False
    if norm is not None and (norm.x.dtype != torch.float32 or norm.x.stride(1) != 1):
        return False
    return a is not None or norm is not None


SKINNY_MAX_ROWS = 128
#: most rows of a step for which the dispatcher lets the few-row kernel normalise the rows itself (every
#: row block of 16 its own rows: 24 launches fewer than with the norm as a kernel of its own)
SKINNY_LN_MAX_ROWS = 128
#: widest row that the few-row kernel normalises in a lane's registers
SKINNY_LN_REGISTER_WIDTH = 1024
PAIR_MIN_ROWS = 256      # the pair kernel's smallest step


def pair_pays(M: int, N: int, K: int) -> bool:
    """Whether a product runs faster by pairs of blocks (one 256-row MMA over two SMs) than on the
    single-block kernel: always from 1536 rows on (measured in whole prefill steps of 2048 rows at
    three model sizes); below that from about one wave of tiles on, or with enough work per output
    (measured alone at widths 768, 1024 and 1600 for the four products of a layer at 256 to 1280 rows)."""
    return M >= 1536 or (M >= PAIR_MIN_ROWS and (M * N >= 3_000_000 or M * N * K >= 3_500_000_000))


def linear_skinny(a, norm, w, bias, out, M, act=ACT_NONE, residual=False, kv=None, split=0) -> bool:
    """The warp-level MMA kernel for steps of at most 128 rows (bfloat16): every SM streams weight
    rows, a few multiply-adds per weight.  ``norm``: the LayerNorm before the product, folded in; ``kv``: (cache layer, block table, row_entry, positions, q_dim) sends keys and
    values straight to the cache; ``split``: blocks of a cluster that split K (0: chosen by the
    library).  False if the kernel does not apply."""
    if M > SKINNY_MAX_ROWS or not _small_inputs_ok(a, norm, w, out):
        return False
    N, K = w.shape
    lib = library()
    if not _can("nib_linear_skinny_supported", M, K, w.stride(0), int(norm is not None), 16 + (_ptr(w) & 15)):
        return False
    ln_args, kv_args = _option_args(norm, kv)
    if tracing():
        _note_linear(a, norm, w, bias, out, M, residual)
    code = lib.nib_linear_skinny(_dt(out), _ptr(a), a.stride(0) if a is not None else 0, _ptr(w), w.stride(0),
                                 _ptr(bias), _ptr(out), out.stride(0), M, N, K, act, int(residual), *ln_args,
                                 *kv_args, int(split), _ptr(status_word()), _stream())
    if code == -2:   # alignment or size not taken
        return False
    _check(code, "linear_skinny")
    return True


def linear_small_tc(a, norm, w, bias, out, M, act=ACT_NONE, residual=False, kv=None, split=True) -> bool:
    """The tensor-core kernel for steps of at most 128 rows with its options: ``norm`` folds the
    LayerNorm before the product into the kernel, ``kv`` sends keys and values straight to the
    cache, ``split`` lets K be split over blocks through scratch.  False if it does not apply."""
    if M > SMALL_STEP_MAX_ROWS or not _small_inputs_ok(a, norm, w, out):
        return False
    N, K = w.shape
    lib = library()
    if not lib.nib_linear_tc_supported(_ptr(a), a.stride(0) if a is not None else 0, _ptr(w), w.stride(0), K):
        return False
    parts, counters = _split_buffers(w.device) if split else (None, None)
    ln_args, kv_args = _option_args(norm, kv)
    if tracing():
        _note_linear(a, norm, w, bias, out, M, residual)
    code = lib.nib_linear_tc_small(_dt(out), _ptr(a), a.stride(0) if a is not None else 0, _ptr(w), w.stride(0),
                                   _ptr(bias), _ptr(out), out.stride(0), M, N, K, act, int(residual), *ln_args,
                                   *kv_args, _ptr(parts), parts.numel() if split else 0, _ptr(counters),
                                   counters.numel() if split else 0, _ptr(status_word()), _stream())
    if code == -2:   # the shape is not taken by the small-step kernel
        return False
    _check(code, "linear_tc_small")
    return True


#: most rows for which the tcgen05 kernel writes keys and values from its epilogue (its swapped orientation)
TC_KV_EPILOGUE_MAX_ROWS = 16


def skinny_pays(M: int, N: int, K: int) -> bool:
    """Whether a product of at most 128 rows goes to the warp-level MMA kernel rather than to tcgen05.
    Measured in whole decode steps at widths 768, 1024 and 1600 (batch 16 to 64): up to 16 rows the MMA
    kernel wins everywhere; up to 32 rows everywhere but the longest rows (K of 4096 and more, split over a
    cluster: GPT-2 medium's second MLP product at 32 rows is 4 % of a step slower here, XL's 20 %) and the
    widest outputs (the head), where its 16-feature tiles read the rows too often; beyond 32 rows while a row
    block holds its rows unsplit.  Flipping one product's choice at a time at 24 to 128 rows and three widths
    moves a step by less than 5 % where the other choice is better and by up to 97 % where it is worse."""
    if M <= 16:
        return True
    if N > 8192 or M > SKINNY_MAX_ROWS:
        return False
    # (33 to 128 rows: while a row block holds its rows unsplit, K up to about a thousand.  The MLP's second
    # product at GPT-2 medium's sizes, K = 4096, on tcgen05 instead: a decode step of 64 rows 1.17 against 1.37 ms)
    return K <= (3072 if M <= 32 else 1088)


def _linear_small(a, norm, w, bias, out, M, act, residual, kv=None) -> bool:
    """Steps of at most 128 rows: the warp-level MMA kernel (with the LayerNorm folded in) where
    ``skinny_pays``, else tcgen05.  Folding the norm into the tcgen05 kernel, or splitting
    K through scratch, costs more round trips than it saves at these sizes, so that kernel is given
    normed rows and is not split here."""
    N, K = w.shape
    mma = skinny_pays(M, N, K)
    if mma:
        # (rows wider than SKINNY_LN_REGISTER_WIDTH are normalised through a buffer per warp in shared memory, which
        # leaves room for one block an SM from 9 rows on: GPT-2 XL at batch 12 to 32 is 2 to 7 % faster with the
        # norm as a kernel of its own there)
        if norm is not None and (M > SKINNY_LN_MAX_ROWS or (K > SKINNY_LN_REGISTER_WIDTH and M > 8)):
            a, norm = norm.materialise(M), None
        if linear_skinny(a, norm, w, bias, out, M, act, residual, kv):
            return True
        if norm is not None:   # too wide or too many rows to be normalised inside the kernel: normalise first
            a, norm = norm.materialise(M), None
            if linear_skinny(a, None, w, bias, out, M, act, residual, kv):
                return True
    if M > TC_KV_EPILOGUE_MAX_ROWS or kv is None:
        return False          # the plain tensor-core call does as well
    if norm is not None:
        a, norm = norm.materialise(M), None
    return linear_small_tc(a, norm, w, bias, out, M, act, residual, kv, split=False)


def linear(a: Optional[torch.Tensor], w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, M: int,
           act: int = ACT_NONE, residual: bool = False, norm: Optional[NormInput] = None) -> None:
    """The matrix product of the model: out[:M] = act(a[:M] . w^T + bias), added to the 32-bit
    ``out`` with ``residual``.  With ``norm`` the activations are LayerNorm of the residual stream
    (``a`` is then None).  bfloat16 runs on the tensor cores where shape and alignment allow (rows
    of 16-byte multiples), else on the CUDA cores; float32 always runs on the CUDA cores in true
    32-bit arithmetic."""
    if _linear_small(a, norm, w, bias, out, M, act, residual):
        return
    if norm is not None:
        a = norm.materialise(M)   # (scratch: a second call for the same rows rewrites the same values)
    if tracing():
        _note_linear(a, None, w, bias, out, M, residual)
    # pairs of blocks on one 256-row MMA (half of the weight tile per SM) beat the single-block kernel
    # by 5 to 40 per cent where there is enough work
    if pair_pays(M, w.shape[0], w.shape[1]) and linear_tc_pair(a, w, bias, out, M, act, residual):
        return
    if linear_tc_supported(a, w):
        linear_tc(a, w, bias, out, M, act, residual)
    else:
        linear_simt(a, w, bias, out, M, act, residual)


def linear_qkv(a: Optional[torch.Tensor], w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, M: int,
               q_dim: int, cache: torch.Tensor, block_table: torch.Tensor, row_entry: torch.Tensor,
               positions: torch.Tensor, status: torch.Tensor, norm: Optional[NormInput] = None) -> bool:
    """The fused q/k/v projection with the cache append in its epilogue: queries to out[:M, :q_dim],
    keys and values to their slots of ``cache``.  Returns False (and does nothing) where no fused
    kernel applies: between 129 rows and the pair kernel's minimum (256), float32, or a shape the
    tensor cores refuse."""
    if cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        return False
    kv = (cache, block_table, row_entry, positions, q_dim)
    # from the pair kernel's smallest step on: it writes the cache from its epilogue, which beats the
    # single-block kernel and a separate append from about 400 rows on and is one launch less
    if M >= PAIR_MIN_ROWS:
        if norm is not None:
            a, norm = norm.materialise(M), None
        return linear_tc_pair(a, w, bias, out, M, kv=kv)
    return _linear_small(a, norm, w, bias, out, M, ACT_NONE, False, kv=kv)


def kv_append(src: torch.Tensor, k_off: int, v_off: int, cache: torch.Tensor, block_table: torch.Tensor,
              row_entry: torch.Tensor, positions: torch.Tensor, T: int, status: torch.Tensor) -> None:
    """Copy the key and value columns of src[:T] to their slots in one cache layer
    [n_pages, 2, n_kv_head, page_size, head_dim]."""
    n_pages, two, n_kv_head, page_size, head_dim = cache.shape
    if two != 2 or not cache.is_contiguous() or cache.dtype != src.dtype or src.stride(1) != 1:
        raise KernelError("kv_append: cache must be contiguous [pages, 2, kv_heads, page, head_dim] of src's dtype")
    _i32(block_table, "block_table")
    if tracing():
        _note("kv_write", "kv_write", (T, 2 * n_kv_head * head_dim, 0), 0.0, 2.0 * T * 2 * n_kv_head * head_dim * src.element_size())
    _check(library().nib_kv_append(_dt(src), _ptr(src), src.stride(0), k_off, v_off, _ptr(cache),
                                   _ptr(block_table), block_table.shape[1], _ptr(row_entry), _ptr(positions),
                                   T, n_kv_head, head_dim, page_size, n_pages, _ptr(status), _stream()),
           "kv_append")


def attention_simt(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, block_table: torch.Tensor,
                   row_entry: torch.Tensor, positions: torch.Tensor, T: int, n_head: int, scale: float,
                   window: int, status: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """Causal attention of T rows of q ([*, n_head * head_dim], any row stride) over one cache layer, with
    the general kernel (any head size up to 256, any page size).  ``rows`` lists the rows to process."""
    n_pages, _, n_kv_head, page_size, head_dim = cache.shape
    if q.dtype != cache.dtype or out.dtype != cache.dtype or q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention: q, out and cache must share a dtype, rows contiguous")
    _check(library().nib_attention_simt(_dt(q), _ptr(q), q.stride(0), _ptr(cache), _ptr(out), out.stride(0),
                                        _ptr(block_table), block_table.shape[1], _ptr(rows), _ptr(row_entry),
                                        _ptr(positions), T, n_head, n_kv_head, head_dim, page_size, n_pages,
                                        float(scale), int(window), _ptr(status), _stream()),
           "attention_simt")


#: blocks of the decode attention that the device holds at once (six an SM): the keys are split so
#: that (rows x heads x splits) stays within it, which also bounds the scratch of the partial results
DECODE_RESIDENT_BLOCKS = 888


_cluster_room: dict = {}


def decode_cluster_room(head_dim: int, cluster: int) -> int:
    """How many clusters of ``cluster`` blocks of the MMA decode attention the device holds at once, asked
    of the runtime once per shape (a cluster's blocks share a GPC: 284 clusters of three, not 296; 142 of
    six).  The splits of a (row, head) are one cluster, and a launch with a cluster too many waits for a
    wave to end: 24 rows of 12 heads took 0.68 ms a step in 3 splits and 0.62 ms in 2."""
    key = (head_dim, cluster)
    got = _cluster_room.get(key)
    if got is None:
        got = int(library().nib_attention_decode_mma_clusters(head_dim, cluster))
        if got < 0:
            raise KernelError(f"attention_decode_mma: the occupancy query failed with CUDA error {-got}")
        _cluster_room[key] = got
    return got


#: numbers of splits that the MMA decode attention runs as one cluster, merging through distributed shared
#: memory instead of global scratch (beyond 8 blocks the cluster size is "non-portable": the kernel is marked
#: as taking it; a lone row at 4,096 keys: 0.331 -> 0.308 ms a step with 16 splits of 256 keys, at 1,024 keys
#: 0.250 -> 0.245 with 16 of 64, one tile a warp)
DECODE_CLUSTER_SPLITS = tuple(range(2, 17))

#: keys per split from which the MMA decode attention gives up the merge inside a cluster for more splits
#: than a cluster holds, merged through scratch (measured at 2 K to 16 K keys, batch 1 to 8: four rows at
#: 16 K keys take 0.67 ms a step in 18 splits through scratch and 0.90 ms in a cluster of 14) ...
DECODE_DEEP_KEYS = 512
#: ... and the fewest such splits: one more than the largest cluster
DECODE_DEEP_SPLITS = 17

def decode_ring_stages(n_blocks: int, n_splits: int, head_dim: int) -> int:
    """How many shared-memory stages per warp the MMA decode attention passes its keys and values through
    (that many tiles in flight per warp beside the one being multiplied; 0: none, the tiles go through
    registers).  The ring pays where the launch fills the device with unsplit rows (measured: -7 to -10 %
    a step at batch 40 to 64, +3 to +7 % at batch 1 to 32, where the keys are split and a block's shared
    memory keeps it from starting beside the kernel ahead).  It is the deepest of two to four stages that
    needs no more waves of blocks than two stages do (shared memory sets how many blocks an SM holds: 40 to 48
    rows of 12 heads take 8 to 9 % less a step with three stages, which still hold them all at once, and
    so do 64 rows of 16 heads, two full waves of four blocks an SM instead of a full and a thin one of six)."""
    if n_splits != 1 or n_blocks < 440:
        return 0
    stage_bytes = 4 * 2 * 16 * head_dim * 2          # four warps, keys and values of a 16-key tile
    by_registers = 6 if head_dim <= 64 else 3

    def waves(stages: int) -> int:
        per_sm = max(1, min(by_registers, (200 * 1024) // (stages * stage_bytes)))
        return -(-n_blocks // (148 * per_sm))

    return max(st for st in (2, 3, 4) if waves(st) <= waves(2))


#: the bfloat16 decode attention on warp-level MMAs where the shape allows (False: always the streaming kernel)
USE_DECODE_MMA = True


def decode_split(n_rows: int, n_head: int, max_keys: int, resident: int = DECODE_RESIDENT_BLOCKS,
                 at_most: int = 0) -> tuple:
    """(chunk, n_splits): keys per split (a multiple of 64) so that the blocks fill the GPU once: six
    blocks an SM are resident, and a block that comes after the first wave runs nearly alone.
    ``at_most``: an upper bound on the number of splits (0: none)."""
    want = max(1, resident // max(1, n_rows * n_head))
    if at_most:
        want = min(want, at_most)
    chunk = max(64, -(-(-(-max_keys // want)) // 64) * 64)
    return chunk, max(1, -(-max_keys // chunk))


def _note_attention(n_q: int, keys_seen: float, kv_rows: float, n_head: int, n_kv_head: int, head_dim: int,
                    itemsize: int) -> None:
    """[queries, keys seen by them in all, width]: per key and head the score (2 hd), the softmax (~5)
    and the weighted sum (2 hd); the queries and outputs, and ``kv_rows`` key and value rows read once."""
    width = n_head * head_dim
    _note("attn", "attn", (n_q, int(keys_seen), width), keys_seen * (4.0 * width + 5.0 * n_head),
          itemsize * (2.0 * n_q * width + 2.0 * kv_rows * n_kv_head * head_dim))


def attention_decode_reserve(workspace, n_head: int, head_dim: int) -> None:
    """Size the decode attention's scratch for good: keys are split only while rows x heads x splits
    fits the resident blocks, so that many partial results (head_dim values, a maximum and a sum
    each) and that many arrival counters are the most any step needs."""
    workspace.reserve("attention.partials", DECODE_RESIDENT_BLOCKS * (head_dim + 2), torch.float32)
    workspace.reserve("attention.arrivals", DECODE_RESIDENT_BLOCKS, torch.int32, zeroed=True)


def attention_decode(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, block_table: torch.Tensor,
                     row_entry: torch.Tensor, positions: torch.Tensor, n_rows: int, n_head: int, scale: float,
                     window: int, status: torch.Tensor, max_keys: int, workspace,
                     rows: Optional[torch.Tensor] = None) -> None:
    """Split-KV attention for rows that are single decoded tokens.  ``max_keys``: the longest key
    range among them; partial results go through ``workspace``.  bfloat16 with a head size of 32, 64,
    96 or 128 runs on the warp-level MMA kernel, everything else (and float32, in true 32-bit
    arithmetic) on the streaming kernel."""
    n_pages, _, n_kv_head, page_size, head_dim = cache.shape
    if q.dtype != cache.dtype or out.dtype != cache.dtype or q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention: q, out and cache must share a dtype, rows contiguous")
    mma = USE_DECODE_MMA and q.dtype == torch.bfloat16 and _can("nib_attention_decode_mma_supported", head_dim, page_size) \
        and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and cache.data_ptr() % 16 == 0
    # (the MMA kernel holds a tile's keys and values in registers: six blocks an SM up to head size 64, three beyond)
    resident = DECODE_RESIDENT_BLOCKS if not mma or head_dim <= 64 else DECODE_RESIDENT_BLOCKS // 2
    # (the MMA kernel merges up to sixteen splits inside a cluster, which costs two trips to memory less
    # than the merge through scratch, until a split has DECODE_DEEP_KEYS keys to walk and the device has
    # room for more splits than a cluster holds: a lone row at 16 K keys takes 0.44 ms a step in 64 splits
    # against 0.72 ms in 8)
    at_most = 0
    if mma:
        at_most = max([c for c in DECODE_CLUSTER_SPLITS if n_rows * n_head <= decode_cluster_room(head_dim, c)], default=1)
        deep = min(resident // max(1, n_rows * n_head), max_keys // (DECODE_DEEP_KEYS // 2))
        if deep >= DECODE_DEEP_SPLITS:
            at_most = deep
    chunk, n_splits = decode_split(n_rows, n_head, max_keys, resident, at_most)
    scratch = counters = None
    if n_splits > 1:
        # (never more than the resident blocks: the same size every step, so that the buffers stay put)
        assert n_rows * n_head * n_splits <= DECODE_RESIDENT_BLOCKS
        scratch = workspace.get("attention.partials", (DECODE_RESIDENT_BLOCKS * (head_dim + 2),), torch.float32)
        counters = workspace.get_zeroed("attention.arrivals", (DECODE_RESIDENT_BLOCKS,), torch.int32)
    if mma:
        _check(library().nib_attention_decode_mma(_ptr(q), q.stride(0), _ptr(cache), _ptr(scratch), _ptr(out),
                                                  out.stride(0), _ptr(block_table), block_table.shape[1], _ptr(rows),
                                                  _ptr(row_entry), _ptr(positions), n_rows, n_head, n_kv_head,
                                                  head_dim, page_size, n_pages, float(scale), int(window), chunk,
                                                  n_splits, _ptr(counters), _ptr(status),
                                                  int(n_splits in DECODE_CLUSTER_SPLITS),
                                                  decode_ring_stages(n_rows * n_head, n_splits, head_dim), _stream()),
               "attention_decode_mma")
        return
    _check(library().nib_attention_decode(_dt(q), _ptr(q), q.stride(0), _ptr(cache), _ptr(scratch), _ptr(out),
                                          out.stride(0), _ptr(block_table), block_table.shape[1], _ptr(rows),
                                          _ptr(row_entry), _ptr(positions), n_rows, n_head, n_kv_head, head_dim,
                                          page_size, n_pages, float(scale), int(window), chunk, n_splits,
                                          _ptr(counters), _ptr(status), _stream()), "attention_decode")


def attention_prefill_tc(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, block_table: torch.Tensor,
                         tiles: torch.Tensor, n_tiles: int, entry_start: torch.Tensor, entry_pos0: torch.Tensor,
                         n_rows: int, n_head: int, scale: float, window: int, status: torch.Tensor) -> None:
    """tcgen05 attention for prompt portions (bfloat16, head size 64): ``tiles`` holds (entry, first
    row within the entry) pairs of 128 rows each; ``q`` holds the step's ``n_rows`` rows."""
    n_pages, _, n_kv_head, page_size, head_dim = cache.shape
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attention_prefill_tc: bfloat16 only")
    if not cache.is_contiguous() or q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention_prefill_tc: contiguous cache layer and rows")
    _check(library().nib_attention_prefill_tc(_ptr(q), q.stride(0), n_rows, _ptr(cache), _ptr(out), out.stride(0),
                                              _ptr(block_table), block_table.shape[1], _ptr(tiles), n_tiles,
                                              _ptr(entry_start), _ptr(entry_pos0), n_head, n_kv_head, head_dim,
                                              page_size, n_pages, float(scale), int(window), _ptr(status),
                                              _stream()), "attention_prefill_tc")


def attention_prefill(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, block_table: torch.Tensor,
                      tiles: torch.Tensor, n_tiles: int, entry_start: torch.Tensor, entry_pos0: torch.Tensor,
                      n_head: int, scale: float, window: int, status: torch.Tensor) -> None:
    """Tiled tensor-core attention for prompt portions: ``tiles`` holds (entry, first row within the
    entry) pairs of 64 rows each."""
    n_pages, _, n_kv_head, page_size, head_dim = cache.shape
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attention_prefill: bfloat16 only")
    _check(library().nib_attention_prefill(_ptr(q), q.stride(0), _ptr(cache), _ptr(out), out.stride(0),
                                           _ptr(block_table), block_table.shape[1], _ptr(tiles), n_tiles,
                                           _ptr(entry_start), _ptr(entry_pos0), n_head, n_kv_head, head_dim,
                                           page_size, n_pages, float(scale), int(window), _ptr(status), _stream()),
           "attention_prefill")


def attention(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, block_table: torch.Tensor, ctx,
              n_head: int, scale: float, window: int, plan) -> None:
    """Causal attention of the step's rows over one cache layer.  ``ctx`` is the step's StepContext,
    ``plan`` says which rows are single decoded tokens and how the prompt portions are cut into
    tiles (``parts.attention.AttentionPlan``).  Single decoded tokens go to the split-KV kernel;
    prompt portions go to the tiled tensor-core kernels in bfloat16 (head sizes 16..128 in steps of
    16) and to the general kernel otherwise."""
    n_pages, _, n_kv_head, page_size, head_dim = cache.shape
    fast_pages = page_size % 16 == 0 and head_dim % 8 == 0 and head_dim <= 128
    traced = tracing()   # (the counts leave a window out: they are those of attention over all keys)
    if not fast_pages:
        if traced:
            _note_attention(ctx.n_rows, plan.decode_keys + plan.prefill_keys, plan.decode_keys + plan.prefill_kv_rows,
                            n_head, n_kv_head, head_dim, q.element_size())
        attention_simt(q, cache, out, block_table, ctx.row_entry, ctx.positions, ctx.n_rows, n_head, scale,
                       window, ctx.status)
        return
    if plan.n_decode:
        keys = plan.max_decode_keys if window <= 0 else min(plan.max_decode_keys, window)
        if traced:
            _note_attention(plan.n_decode, plan.decode_keys, plan.decode_keys, n_head, n_kv_head, head_dim,
                            q.element_size())
        attention_decode(q, cache, out, block_table, ctx.row_entry, ctx.positions, plan.n_decode, n_head, scale,
                         window, ctx.status, keys, ctx.workspace, plan.decode_rows)
    if plan.n_prefill_rows:
        if traced:
            _note_attention(plan.n_prefill_rows, plan.prefill_keys, plan.prefill_kv_rows, n_head, n_kv_head, head_dim,
                            q.element_size())
        if q.dtype == torch.bfloat16 and _can("nib_attention_prefill_tc_supported", head_dim, page_size) \
                and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.stride(0) % 8 == 0 \
                and out.data_ptr() % 16 == 0:
            attention_prefill_tc(q, cache, out, block_table, plan.wide_tiles, plan.n_wide_tiles, ctx.entry_start,
                                 ctx.entry_pos0, ctx.n_rows, n_head, scale, window, ctx.status)
        elif q.dtype == torch.bfloat16 and _can("nib_attention_prefill_supported", head_dim) \
                and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0:
            attention_prefill(q, cache, out, block_table, plan.tiles, plan.n_tiles, ctx.entry_start, ctx.entry_pos0,
                              n_head, scale, window, ctx.status)
        else:
            # (portions alone: all of the step's rows, those of no request among them, which the kernel leaves out;
            # the launch then depends on the step's shape only, as a graph needs it)
            attention_simt(q, cache, out, block_table, ctx.row_entry, ctx.positions,
                           plan.n_prefill_rows if plan.n_decode else ctx.n_rows, n_head, scale, window, ctx.status,
                           plan.prefill_rows)


_SRC_CODES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def convert_rows(src: torch.Tensor, src_dtype: torch.dtype, rows: int, cols: int, dst: torch.Tensor, r0: int,
                 transpose: bool) -> None:
    """Loading: ``src`` holds the raw bytes of ``rows`` x ``cols`` values as a checkpoint stores them;
    they are converted to ``dst``'s dtype and written to dst[r0:r0 + rows, :] or, transposed, to
    dst[:, r0:r0 + rows]."""
    if src_dtype not in _SRC_CODES or not dst.is_contiguous() or dst.dim() != 2:
        raise KernelError("convert: 16- or 32-bit floats into a contiguous matrix")
    _check(library().nib_convert(_SRC_CODES[src_dtype], _ptr(src), rows, cols, _dt(dst), _ptr(dst), dst.stride(0),
                                 int(r0), int(bool(transpose)), _stream()), "convert")


def argmax(logits: torch.Tensor, out: torch.Tensor, n_rows: int) -> None:
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("argmax: logits must be float32 with contiguous rows")
    _i32(out, "out")
    if tracing():
        _note("sample", "sample", (n_rows, logits.shape[1], 0), n_rows * logits.shape[1], 4.0 * n_rows * logits.shape[1])
    _check(library().nib_argmax(_ptr(logits), logits.stride(0), n_rows, logits.shape[1], _ptr(out), _stream()),
           "argmax")


def sample(logits: torch.Tensor, n_rows: int, row_slot: torch.Tensor, temperature: torch.Tensor,
           top_k: torch.Tensor, rng_state: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor,
           last_token: Optional[torch.Tensor] = None, teams: bool = True) -> None:
    """One token per row.  ``temperature``, ``top_k`` and ``rng_state`` are per-slot arrays and
    ``row_slot`` names each row's slot: greedy where the slot's temperature <= 0, else
    temperature / top-k sampling that advances the slot's xorshift64* word.  ``last_token``: a
    per-slot array that also receives the tokens (for the next step's embedding).  ``teams``: launch
    clusters of blocks that share a sampled row's passes over the vocabulary (False when every row
    is known to be greedy; the tokens are the same either way).  ``scratch``: two int64 words per
    row that the kernel finds zero and leaves zero (the caller owns them, so that they stay where
    they are for as long as a captured launch may use them)."""
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 with contiguous rows")
    if rng_state.dtype != torch.int64 or temperature.dtype != torch.float32:
        raise KernelError("sample: rng_state must be int64 words, temperature float32")
    _i32(row_slot, "row_slot"); _i32(top_k, "top_k"); _i32(out, "out")
    if scratch.dtype != torch.int64 or scratch.numel() < 2 * n_rows or out.numel() < n_rows:
        raise KernelError("sample: scratch must hold two int64 words per row, out one int32")
    if tracing():
        _note("sample", "sample", (n_rows, logits.shape[1], 0), n_rows * logits.shape[1], 4.0 * n_rows * logits.shape[1])
    _check(library().nib_sample(_ptr(logits), logits.stride(0), n_rows, logits.shape[1], _ptr(row_slot),
                                _ptr(temperature), _ptr(top_k), _ptr(rng_state), _ptr(out),
                                _ptr(last_token), _ptr(scratch), int(bool(teams)), _stream()), "sample")
