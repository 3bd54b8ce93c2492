"""The kernels as Python functions over torch tensors.

Every function launches hand-written CUDA from `csrc/` on the current stream through
ctypes. There is no CPU path and no library fallback: without a CUDA device, or when a
library cannot be built or loaded, a call raises. A kernel that cannot take a size
refuses it with the message its entry point stored; nothing is retried elsewhere.

Tensors are contiguous; activations and matrices are float32 or bfloat16, biases and
norm weights float32, indices int32, logits float32.
"""

from __future__ import annotations

import ctypes
import re
from ctypes import c_float, c_int, c_void_p

import torch

from . import build

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
_libs: dict[str, ctypes.CDLL] = {}

# Kernel launches made through this module since import (read by the measurement script).
launches = 0


# True when the libraries are the checked build (PAE_BOUNDS=1: see kernels/build.py). The kernels
# then compare every slot, block-table index and page id with the pool before using it; the
# limits are handed to a library whenever they change, which a recorded graph cannot follow, so
# the runner records none in this mode.
bounds_checked = build.BOUNDS
_bounds_set: dict[str, tuple] = {}


class KernelError(RuntimeError):
    pass


def _set_bounds(name: str, pages_of: torch.Tensor | None) -> None:
    """Checked build only: tells library `name` how many pages the pool of `pages_of` has."""
    if not bounds_checked or pages_of is None:
        return
    flag = _error_flag(pages_of.device)
    limits = (int(pages_of.shape[0]), flag.data_ptr())
    if _bounds_set.get(name) != limits:
        lib = _lib(name)
        code = lib.pae_set_bounds(ctypes.c_longlong(limits[0]), c_void_p(limits[1]))
        if code != 0:
            raise KernelError(lib.pae_last_error().decode(errors="replace"))
        _bounds_set[name] = limits


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError(
            "paged_attention_engine_b200 runs on a CUDA device only (sm_100a); no device is visible "
            "and there is no CPU path"
        )


_SIGNATURE = re.compile(r"PAE_EXPORT\s+([\w\s\*]+?)\s*\b(pae_\w+)\s*\(([^)]*)\)")


def _ctype_of(declaration: str):
    if "*" in declaration:
        return ctypes.c_char_p if declaration.strip().startswith("const char") and declaration.strip().endswith("*") else c_void_p
    if "long long" in declaration:
        return ctypes.c_longlong
    if "float" in declaration:
        return c_float
    return c_int


def _declare_signatures(lib: ctypes.CDLL, name: str) -> None:
    """Tells ctypes the argument and result types of the family's entry points, read from their
    declarations in the sources (`PAE_EXPORT <type> pae_name(<arguments>)`): a call then takes plain
    Python integers, floats and addresses, which is quicker than wrapping each in a ctypes object,
    and an address is never cut to 32 bits."""
    for source in build.FAMILIES[name]:
        text = (build.CSRC / source).read_text()
        for result, function, arguments in _SIGNATURE.findall(text):
            entry = getattr(lib, function, None)
            if entry is None:
                continue
            arguments = arguments.strip()
            entry.argtypes = [] if arguments in ("", "void") else [
                c_void_p if "*" in a else _ctype_of(a) for a in arguments.split(",")]
            entry.restype = _ctype_of(result)


def _lib(name: str) -> ctypes.CDLL:
    lib = _libs.get(name)
    if lib is None:
        require_cuda()
        path = build.ensure_built([name])[name]
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as exc:
            raise KernelError(f"cannot load {path}: {exc}") from exc
        lib.pae_last_error.restype = ctypes.c_char_p
        _declare_signatures(lib, name)
        _libs[name] = lib
    return lib


def preload(names: list[str]) -> None:
    """Builds (in parallel) and loads the given families."""
    require_cuda()
    build.ensure_built([n for n in names if n not in _libs])
    for n in names:
        _lib(n)


def _check(lib: ctypes.CDLL, code: int, count: int = 1) -> None:
    global launches
    launches += count
    if code != 0:
        raise KernelError(lib.pae_last_error().decode(errors="replace") + f" (code {code})")


def _ptr(t: torch.Tensor | None):
    """A tensor's address as an integer (the entry points' pointer arguments are declared)."""
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


_get_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current stream's handle (asked for at every launch: the quick way when torch has it)."""
    if _raw_stream is not None and _get_device is not None:
        return _raw_stream(_get_device())
    return torch.cuda.current_stream().cuda_stream


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not supported (float32 or bfloat16)") from None


def _need(t: torch.Tensor, what: str, dtype=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what} is not on a CUDA device")
    if not t.is_contiguous():
        raise KernelError(f"{what} is not contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what} is {t.dtype}, {dtype} is needed")


# ----------------------------------------------------------------------------------- #

class PendingSum:
    """A split-K product whose float32 partial sums [splits, M, N] have not been added up yet.

    `linear` returns one for a step of few tokens. `rms_norm`, `silu_mul` and
    `rotary_qk_cache_write` add the splits up inside their own kernel (bias and residual
    included), which saves a launch; anything else calls `materialized`, which runs the
    stand-alone reduction once and keeps its result in `value`."""

    def __init__(self, partial, bias, residual, out_dtype):
        self.partial = partial
        self.bias = bias
        self.residual = residual
        self.dtype = out_dtype
        self.value = None

    @property
    def shape(self):
        return self.partial.shape[1:]

    @property
    def device(self):
        return self.partial.device


class PendingNorm:
    """RMSNorm(x) * weight of a step of few tokens that has not been computed: `rms_norm` returns
    one, and the products that can (`qkv_projection`, `linear_swiglu`, `linear` without bias) apply
    the norm while they stage their operand, which saves the norm's own launch; anything else
    calls `materialized`, which runs the norm's kernel once and keeps its result in `value`."""

    def __init__(self, x: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
        self.x = x
        self.weight = weight
        self.eps = eps
        self.value = None

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype

    @property
    def device(self):
        return self.x.device


def materialized(x):
    """The tensor that `x` stands for (x itself unless it is a PendingSum or a PendingNorm)."""
    if isinstance(x, PendingNorm):
        if x.value is None:
            x.value = _rms_norm_now(x.x, x.weight, x.eps)
        return x.value
    if not isinstance(x, PendingSum):
        return x
    if x.value is None:
        splits, m, n = x.partial.shape
        out = torch.empty((m, n), dtype=x.dtype, device=x.partial.device)
        lib = _lib("gemm_tcgen05")
        _check(lib, lib.pae_reduce_splits(_ptr(out), _ptr(x.partial), _ptr(x.bias), _ptr(x.residual), splits,
                                          m, n, (1 if x.dtype == torch.float32 else 0), _stream()))
        x.value = out
    return x.value


def gather_rows(x, rows: torch.Tensor) -> torch.Tensor:
    x = materialized(x)
    _need(x, "gather_rows: x")
    _need(rows, "gather_rows: rows", torch.int32)
    out = torch.empty((rows.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    lib = _lib("elementwise")
    _check(lib, lib.pae_gather_rows(_ptr(out), _ptr(x), _ptr(rows), (rows.numel()), x.shape[0],
                                    x.shape[1], (_code(x)), _stream()))
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, feedback=None) -> torch.Tensor:
    """Rows of `table` for the token ids. With `feedback` = (last_token, state_slot, seq_index) a
    negative id stands for the token that the request sampled in the step before, read from
    last_token[state_slot[seq_index[t]]] on the device."""
    if feedback is None:
        return gather_rows(table, ids)
    last_token, state_slot, seq_index = feedback
    _need(table, "embedding: table")
    for name, t in (("ids", ids), ("last_token", last_token), ("state_slot", state_slot), ("seq_index", seq_index)):
        _need(t, f"embedding: {name}", torch.int32)
    out = torch.empty((ids.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
    lib = _lib("elementwise")
    _check(lib, lib.pae_embedding_feedback(_ptr(out), _ptr(table), _ptr(ids), _ptr(last_token), _ptr(state_slot),
                                           _ptr(seq_index), (ids.numel()), table.shape[0],
                                           table.shape[1], (_code(table)), _stream()))
    return out


def scatter_tokens(last_token, tokens, logit_rows, seq_index, state_slot) -> None:
    """last_token[state_slot[seq_index[logit_rows[r]]]] = tokens[r]: the sampled tokens stay on the
    device where the next step's embedding finds them."""
    for name, t in (("last_token", last_token), ("tokens", tokens), ("logit_rows", logit_rows),
                    ("seq_index", seq_index), ("state_slot", state_slot)):
        _need(t, f"scatter_tokens: {name}", torch.int32)
    lib = _lib("elementwise")
    _check(lib, lib.pae_scatter_tokens(_ptr(last_token), _ptr(tokens), _ptr(logit_rows), _ptr(seq_index),
                                       _ptr(state_slot), (tokens.numel()), _stream()))


def rms_norm(x, weight: torch.Tensor, eps: float) -> torch.Tensor:
    _need(weight, "rms_norm: weight", torch.float32)
    if weight.numel() != x.shape[-1]:
        raise KernelError(f"rms_norm: weight of {weight.numel()} for rows of {x.shape[-1]}")
    if isinstance(x, PendingSum) and x.value is None:
        splits, m, n = x.partial.shape
        value = torch.empty((m, n), dtype=x.dtype, device=x.device)
        normed = torch.empty_like(value)
        lib = _lib("fused_decode")
        _check(lib, lib.pae_splitk_rms_norm(_ptr(normed), _ptr(value), _ptr(x.partial), splits, _ptr(x.bias),
                                            _ptr(x.residual), _ptr(weight), m, n, eps,
                                            _DTYPE_CODE[x.dtype], _stream()))
        x.value = value
        return normed
    x = materialized(x)
    _need(x, "rms_norm: x")
    if x.dim() == 2 and _few_tokens(x, x.shape[-1], normed=True):
        return PendingNorm(x, weight, eps)       # the product that follows applies it
    return _rms_norm_now(x, weight, eps)


def _rms_norm_now(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    out = torch.empty_like(x)
    lib = _lib("elementwise")
    rows = x.numel() // x.shape[-1] if x.numel() else 0
    _check(lib, lib.pae_rms_norm(_ptr(out), _ptr(x), _ptr(weight), rows, (x.shape[-1]), eps,
                                 (_code(x)), _stream()))
    return out


# A step of few tokens (decoding) runs a product as one kernel that leaves finished output
# (csrc/gemv_mma.cu: a warp owns 16 weight rows and the whole K, so no partial sums are left for a
# kernel of their own, and the norm before and the rotation, SiLU x up or residual after run
# inside the product) where that is the faster way: where all blocks of that kernel run at once.
# False sends every product to the tcgen05 kernels and their summing kernels (tests compare the
# two); `few_token_products_everywhere` sends every product that the kernels can take at all.
use_few_token_products = True
few_token_products_everywhere = False
FEW_TOKENS_MAX = 24
QKV_KIND, RESIDUAL_KIND, GATE_UP_KIND = 0, 1, 2
# Up to how many tokens a kind of product is faster there than as a tcgen05 product with its summing
# kernel (measured at the 1536-wide sizes, 24 tokens: q|k|v 6.7 against 8.4 us, o 4.9 against 6.5,
# gate|up 14.3 against 16.5; down, whose warps bring the tokens' operand through their rings once
# each, 10.2 against 9.6. A decode step of 24 requests: 1.63 against 1.75 ms; with kernels for 32
# tokens a step of 28 or 32 was no faster, 1.92 against 1.89 and 2.01 against 1.99 ms, and they are not built).
FEW_TOKENS_MAX_QKV = 24
FEW_TOKENS_MAX_RESIDUAL = 24          # while K is short ...
FEW_TOKENS_MAX_RESIDUAL_LONG_K = 16   # ... and from K = 2,048 on
FEW_TOKENS_MAX_GATE_UP = 24


def _few_tokens(x: torch.Tensor, k: int, normed: bool = False, kind: int = GATE_UP_KIND, n: int = 16) -> bool:
    """Whether a product of `kind` over x [tokens, K] with `n` weight rows runs as a few-token
    kernel; `normed`: with the RMSNorm of x folded in (the normed operand has to fit shared memory)."""
    if not (use_few_token_products and use_tensor_cores and x.dtype == torch.bfloat16 and x.dim() == 2
            and 0 < x.shape[0] <= FEW_TOKENS_MAX and x.data_ptr() % 16 == 0):
        return False
    if k < 64 or k % 64:        # not for these kernels: their library is not even built for such a model
        return False
    answer = _lib("gemv_mma").pae_linear_few_tokens_supports(kind, x.shape[0], n, k, 1 if normed else 0)
    if few_token_products_everywhere:
        return answer >= 1
    most = (FEW_TOKENS_MAX_QKV if kind == QKV_KIND else FEW_TOKENS_MAX_GATE_UP if kind == GATE_UP_KIND
            else FEW_TOKENS_MAX_RESIDUAL if k < SWAPPED_LONG_K else FEW_TOKENS_MAX_RESIDUAL_LONG_K)
    return answer == 2 and x.shape[0] <= most


def _norm_of(x):
    """(input tensor, norm weight or None, eps) of an operand that may be a PendingNorm."""
    if isinstance(x, PendingNorm) and x.value is None:
        return x.x, x.weight, x.eps
    return materialized(x), None, 0.0


# The bfloat16 products run on the tcgen05 kernels when the shape allows; set to False to
# send everything to the CUDA-core kernel (tests compare the two).
use_tensor_cores = True
# Whether a split-K product is summed inside the kernel that consumes it (tests compare both).
fuse_split_sums = True
SWAPPED_MAX_TOKENS = 64
# ... and up to this many where K is long (2,048 and more): the swapped product's blocks then
# have enough of K each, and it stays ahead of the many-token kernel with its K shared out in
# planes (128 tokens at the 3584-wide sizes: q|k|v 19.8 against 22.5 us, o 16.3 against 19.2; down of
# the 1536-wide sizes, K = 8960: 14.0 against 16.3; its q|k|v and o, K = 1536: 14.7 and 10.5 against 12.4 and 9.7).
SWAPPED_MAX_TOKENS_LONG_K = 128
SWAPPED_LONG_K = 2048


def _swapped(m: int, k: int) -> bool:
    """Whether a product of m tokens over K takes the swapped split-K kernel."""
    return m <= SWAPPED_MAX_TOKENS or (m <= SWAPPED_MAX_TOKENS_LONG_K and k >= SWAPPED_LONG_K)
# gate|up takes the many-token kernel (SiLU x up in its epilogue, no split of K, tiles of 128 tokens)
# from 33 tokens on: at 64 tokens 16.8 against 21.9 us at the 1536-wide sizes and 52.2 against
# 61.1 us at the 3584-wide ones; at 32 tokens 18.7 against 17.6 and 51.6 against 53.4, below that the
# swapped product and the kernel that adds its two splits are faster.
SWIGLU_SWAPPED_MAX_TOKENS = 32

_error_flags: dict[int, torch.Tensor] = {}


def _error_flag(device: torch.device) -> torch.Tensor:
    index = device.index if device.index is not None else torch.cuda.current_device()
    flag = _error_flags.get(index)
    if flag is None:
        with torch.inference_mode(False):      # an ordinary tensor, whoever asks first: it is cleared from anywhere
            flag = torch.zeros(1, dtype=torch.int32, device=device)
        _error_flags[index] = flag
    return flag


def error_flag(device) -> torch.Tensor:
    """The device's error word (int32 [1]): 0, or the role code of a wait that gave up. The
    generation path copies it to the host beside the sampled tokens and hands it to
    `raise_for_error_word`, so that a step whose kernel gave up never yields tokens silently."""
    return _error_flag(torch.device(device))


def raise_for_error_word(code: int, device) -> None:
    """Raises (and clears the device's word) when `code`, a copy of the error word, is not 0."""
    if code:
        _error_flag(torch.device(device)).zero_()
        index = torch.device(device).index
        if int(code) >= 100:
            what = {101: "a slot beyond the pool", 102: "a block-table index beyond the table's width",
                    103: "a page id that is negative or beyond the pool"}.get(int(code), "an index out of range")
            raise KernelError(f"a kernel on device {index} met {what} (bounds code {int(code)}); the access was skipped")
        raise KernelError(
            f"a tensor-core kernel on device {index} gave up waiting on an mbarrier (role code {int(code)}; 8: a warp of a "
            "few-token product, others: the roles of a tcgen05 kernel); "
            "its output is not valid"
        )


def check_device_errors() -> None:
    """Raises if a kernel gave up on a bounded wait since the last check (synchronises)."""
    for index, flag in _error_flags.items():
        raise_for_error_word(int(flag.item()), flag.device)


def _tensor_core_shape(x, weight, residual, out_dtype) -> bool:
    return (
        use_tensor_cores
        and x.dtype == torch.bfloat16
        and weight.dtype == torch.bfloat16
        and x.shape[1] % 8 == 0
        and x.data_ptr() % 16 == 0
        and weight.data_ptr() % 16 == 0
    )


def linear(x, weight, bias=None, residual=None, out_dtype=None) -> torch.Tensor:
    """x [M, K] . weight [N, K]^T (+ bias [N], float32) (+ residual [M, N]) -> [M, N]."""
    if (bias is None and out_dtype in (None, torch.bfloat16) and weight.dtype == torch.bfloat16 and weight.dim() == 2
            and weight.data_ptr() % 16 == 0 and weight.shape[0] <= 65536):
        source, norm_weight, eps = _norm_of(x)
        if (_few_tokens(source, weight.shape[1], norm_weight is not None, RESIDUAL_KIND, weight.shape[0]) and source.dim() == 2 and source.shape[1] == weight.shape[1]
                and source.is_contiguous() and weight.is_contiguous()):
            residual_now = materialized(residual)
            m, n = source.shape[0], weight.shape[0]
            if residual_now is not None:
                _need(residual_now, "linear: residual", torch.bfloat16)
                if tuple(residual_now.shape) != (m, n):
                    raise KernelError(f"linear: residual is {tuple(residual_now.shape)}, the product is [{m}, {n}]")
            out = torch.empty((m, n), dtype=torch.bfloat16, device=source.device)
            lib = _lib("gemv_mma")
            _check(lib, lib.pae_linear_few_tokens(_ptr(out), _ptr(source), _ptr(weight), _ptr(residual_now), _ptr(norm_weight),
                                                  eps, m, n, weight.shape[1], _ptr(_error_flag(source.device)), _stream()))
            return out
    x = materialized(x)
    residual = materialized(residual)
    _need(x, "linear: x")
    _need(weight, "linear: weight")
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"linear: x is [{m}, {k}], weight is {tuple(weight.shape)}")
    out_dtype = out_dtype or x.dtype
    if bias is not None:
        _need(bias, "linear: bias", torch.float32)
    if residual is not None:
        _need(residual, "linear: residual", out_dtype)
        if tuple(residual.shape) != (m, n):
            raise KernelError(f"linear: residual is {tuple(residual.shape)}, the product is [{m}, {n}]")
    if m == 0:
        return torch.empty((m, n), dtype=out_dtype, device=x.device)
    if _tensor_core_shape(x, weight, residual, out_dtype):
        return _linear_tensor_cores(x, weight, bias, residual, out_dtype, m, n, k)
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    lib = _lib("gemm_simt")
    _check(lib, lib.pae_linear_simt(_ptr(out), _ptr(x), _ptr(weight), _ptr(bias), _ptr(residual), m, n,
                                    k, (_code(x)), (_code(weight)), _DTYPE_CODE[out_dtype],
                                    _stream()))
    return out


def _linear_tensor_cores(x, weight, bias, residual, out_dtype, m, n, k) -> torch.Tensor:
    lib = _lib("gemm_tcgen05")
    flag = _error_flag(x.device)
    out_f32 = (1 if out_dtype == torch.float32 else 0)
    if _swapped(m, k):
        # Few tokens: weight rows fill the MMA's 128 rows, K is split, partial sums are
        # float32 scratch that the reduction (or nothing, for one split) turns into the output.
        splits = lib.pae_linear_swapped_splits(n, k)
        partial = torch.empty((splits, m, n), dtype=torch.float32, device=x.device)
        _check(lib, lib.pae_linear_tcgen05_swapped(_ptr(partial), _ptr(x), _ptr(weight), m, n, k,
                                                   _ptr(flag), _stream()))
        if splits == 1 and bias is None and residual is None and out_dtype == torch.float32:
            return partial[0]
        pending = PendingSum(partial, bias, residual, out_dtype)
        return pending if fuse_split_sums else materialized(pending)
    planes = lib.pae_linear_tcgen05_plane_count(m, n, k)
    if planes > 1:
        # Few output tiles and a long K (a down projection for a few hundred tokens): each
        # tile's K is shared out over several blocks, whose float32 planes are added up later.
        partial = torch.empty((planes, m, n), dtype=torch.float32, device=x.device)
        _check(lib, lib.pae_linear_tcgen05_planes(_ptr(partial), _ptr(x), _ptr(weight), m, n, k,
                                                  planes, _ptr(flag), _stream()))
        pending = PendingSum(partial, bias, residual, out_dtype)
        return pending if fuse_split_sums else materialized(pending)
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    _check(lib, lib.pae_linear_tcgen05(_ptr(out), _ptr(x), _ptr(weight), _ptr(bias), _ptr(residual), m, n,
                                       k, out_f32, _ptr(flag), _stream()))
    return out


def rotary_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    _need(positions, "rotary_table: positions", torch.int32)
    _need(inv_freq, "rotary_table: inv_freq", torch.float32)
    half = inv_freq.numel()
    table = torch.empty((positions.numel(), 2 * half), dtype=torch.float32, device=positions.device)
    lib = _lib("elementwise")
    _check(lib, lib.pae_rotary_table(_ptr(table), _ptr(positions), _ptr(inv_freq), (positions.numel()),
                                     half, _stream()))
    return table


def rotary_qk_cache_write(qkv, table, slots, keys, values, num_heads, num_kv_heads, head_dim, page_size) -> torch.Tensor:
    """Rotates q and k of the fused projection's output (in place), writes k and v to their
    pages, and returns the [tokens, (heads + 2 kv_heads) * head_dim] tensor."""
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape[1] != width:
        raise KernelError(f"rotary_qk_cache_write: qkv rows of {qkv.shape[1]} for {num_heads}+2x{num_kv_heads} heads of {head_dim}")
    tokens = qkv.shape[0]
    if table is not None:
        _need(table, "rotary_qk_cache_write: table", torch.float32)
        if tuple(table.shape) != (tokens, head_dim):
            raise KernelError(f"rotary_qk_cache_write: table is {tuple(table.shape)}, [{tokens}, {head_dim}] is needed")
    if slots is not None:
        _need(slots, "rotary_qk_cache_write: slots", torch.int32)
        _need(keys, "rotary_qk_cache_write: keys", qkv.dtype)
        _need(values, "rotary_qk_cache_write: values", qkv.dtype)
    key_ptr = _ptr(keys if slots is not None else None)
    value_ptr = _ptr(values if slots is not None else None)
    if isinstance(qkv, PendingSum) and qkv.value is None and qkv.residual is None:
        splits = qkv.partial.shape[0]
        out = torch.empty((tokens, width), dtype=qkv.dtype, device=qkv.device)
        lib = _lib("fused_decode")
        _set_bounds("fused_decode", keys if slots is not None else None)
        _check(lib, lib.pae_splitk_rotary_cache_write(
            _ptr(out), _ptr(qkv.partial), splits, _ptr(qkv.bias), _ptr(table), _ptr(slots), key_ptr, value_ptr,
            tokens, num_heads, num_kv_heads, head_dim, page_size,
            _DTYPE_CODE[qkv.dtype], _stream()))
        qkv.value = out
        return out
    qkv = materialized(qkv)
    _need(qkv, "rotary_qk_cache_write: qkv")
    lib = _lib("elementwise")
    _set_bounds("elementwise", keys if slots is not None else None)
    _check(lib, lib.pae_rotary_qk_cache_write(
        _ptr(qkv), _ptr(table), _ptr(slots), key_ptr, value_ptr, tokens, num_heads, num_kv_heads,
        head_dim, page_size, (_code(qkv)), _stream()))
    return qkv


# Whether q|k|v of a prompt's portion is finished (bias, rotation, page write) by the product's own epilogue.
fuse_qkv_epilogue = True


def qkv_projection(x, weight, bias, table, slots, keys, values, num_heads, num_kv_heads, head_dim, page_size) -> torch.Tensor:
    """`rotary_qk_cache_write(linear(x, weight, bias), ...)`: q|k|v of the step's tokens, q and k
    rotated, k and v written to their pages. For more than 64 tokens on the tensor-core path it
    is one kernel (the product's epilogue rotates and writes); otherwise the two calls, which
    for few tokens fuse the other way round (the split sum runs inside the rotation kernel)."""
    m, k = x.shape
    n = weight.shape[0]
    source, norm_weight, eps = _norm_of(x)
    if (_few_tokens(source, k, norm_weight is not None, QKV_KIND, n) and weight.dtype == torch.bfloat16 and weight.is_contiguous() and weight.data_ptr() % 16 == 0
            and n == (num_heads + 2 * num_kv_heads) * head_dim and weight.shape[1] == k and head_dim % 16 == 0
            and (slots is None or (keys.dtype == torch.bfloat16 and values.dtype == torch.bfloat16))):
        _need(source, "qkv_projection: x")
        if bias is not None:
            _need(bias, "qkv_projection: bias", torch.float32)
        if table is not None:
            _need(table, "qkv_projection: table", torch.float32)
            if tuple(table.shape) != (m, head_dim):
                raise KernelError(f"qkv_projection: table is {tuple(table.shape)}, [{m}, {head_dim}] is needed")
        if slots is not None:
            _need(slots, "qkv_projection: slots", torch.int32)
            _need(keys, "qkv_projection: keys", torch.bfloat16)
            _need(values, "qkv_projection: values", torch.bfloat16)
        out = torch.empty((m, n), dtype=torch.bfloat16, device=source.device)
        lib = _lib("gemv_mma")
        _set_bounds("gemv_mma", keys if slots is not None else None)
        _check(lib, lib.pae_qkv_few_tokens(
            _ptr(out), _ptr(source), _ptr(weight), _ptr(bias), _ptr(norm_weight), eps, _ptr(table), _ptr(slots),
            _ptr(keys if slots is not None else None), _ptr(values if slots is not None else None), m, num_heads,
            num_kv_heads, head_dim, page_size, k, _ptr(_error_flag(source.device)), _stream()))
        return out
    x = materialized(x)
    if (fuse_qkv_epilogue and not _swapped(m, k) and n >= 256 and n == (num_heads + 2 * num_kv_heads) * head_dim
            and weight.shape[1] == k and not isinstance(x, PendingSum) and _tensor_core_shape(x, weight, None, x.dtype)
            and (slots is None or (keys.dtype == torch.bfloat16 and values.dtype == torch.bfloat16))):
        lib = _lib("gemm_tcgen05")
        # With so few output tiles that K is shared out over blocks, the sum of the planes rotates and writes.
        if lib.pae_linear_rotary_tcgen05_supports(head_dim) and lib.pae_linear_tcgen05_plane_count(m, n, k) == 1:
            _need(x, "qkv_projection: x")
            _need(weight, "qkv_projection: weight")
            if bias is not None:
                _need(bias, "qkv_projection: bias", torch.float32)
                if bias.numel() != n:
                    raise KernelError(f"qkv_projection: bias of {bias.numel()} for {n} columns")
            if table is not None:
                _need(table, "qkv_projection: table", torch.float32)
                if tuple(table.shape) != (m, head_dim):
                    raise KernelError(f"qkv_projection: table is {tuple(table.shape)}, [{m}, {head_dim}] is needed")
            if slots is not None:
                _need(slots, "qkv_projection: slots", torch.int32)
                _need(keys, "qkv_projection: keys", torch.bfloat16)
                _need(values, "qkv_projection: values", torch.bfloat16)
            out = torch.empty((m, n), dtype=x.dtype, device=x.device)
            _set_bounds("gemm_tcgen05", keys if slots is not None else None)
            _check(lib, lib.pae_linear_rotary_tcgen05(
                _ptr(out), _ptr(x), _ptr(weight), _ptr(bias), _ptr(table), _ptr(slots),
                _ptr(keys if slots is not None else None), _ptr(values if slots is not None else None), m,
                num_heads, num_kv_heads, head_dim, page_size, k,
                _ptr(_error_flag(x.device)), _stream()))
            return out
    return rotary_qk_cache_write(linear(x, weight, bias), table, slots, keys, values, num_heads, num_kv_heads, head_dim,
                                 page_size)


def decode_slicing(seqs: int, kv_heads: int, max_kv_len: int, most: int | None = None, wave_blocks: int = 444,
                   slices_per_block: int = 4) -> tuple[int, int]:
    """(keys per slice, slices) for the decode kernel. A block is `slices_per_block` slices of
    one (request, kv head) pair, and `wave_blocks` blocks run at one time: as many slices as
    keep all blocks in that one wave (a second, partly filled wave costs as much as a full
    one), at most `most`, each of at least 32 keys in steps of 16. A warp walks its slice one
    trip to memory after the other, so short slices are what makes few requests fast: up to 96
    for contexts of up to 6,144 keys (batch 1 at context 4,096: 0.940 -> 0.915 ms a step, batch 8:
    1.032 -> 1.024), beyond that up to 192 of at least 64 keys (batch 1 at context 32,768: 1.72 ms
    with 64 slices, 1.43 with 96, 1.24 with 192, 1.21 with 256, 1.25 with 384; batch 4 at 16,384:
    1.33, 1.20, 1.21; eight requests and more fill the wave with fewer slices anyway). The merge
    holds 96 slices' partial outputs in registers and walks the rest one by one."""
    if most is None:
        most = 96 if max_kv_len <= 96 * 64 else min(192, max_kv_len // 64)
    pairs = max(1, seqs * kv_heads)
    blocks_per_pair = max(1, wave_blocks // pairs)
    wanted = max(1, min(most, slices_per_block * blocks_per_pair))
    slice_keys = max(32, -(-(-(-max_kv_len // wanted)) // 16) * 16)
    while -(-(max_kv_len + 15) // slice_keys) > wanted:
        slice_keys += 16
    return slice_keys, -(-(max_kv_len + 15) // slice_keys)


use_tcgen05_attention = True
TCGEN05_ATTENTION_MIN_TOKENS = 64


def _decode_attention(lib, out, qkv, keys, values, block_table, q_start, kv_len, seqs, singles, num_heads,
                      num_kv_heads, head_dim, page_size, max_kv_len, scale, window) -> None:
    """The requests that bring one token: sliced over their keys, then merged."""
    count = seqs if singles < 0 else singles
    wave = lib.pae_decode_blocks_per_wave(head_dim)
    slice_keys, max_slices = decode_slicing(count, num_kv_heads, max_kv_len, wave_blocks=wave,
                                            slices_per_block=lib.pae_decode_slices_per_block())
    floats = lib.pae_decode_scratch_floats(seqs, num_heads, head_dim, max_slices)
    scratch = torch.empty(floats, dtype=torch.float32, device=qkv.device)
    launches = 2
    _set_bounds("attention_mma", keys)
    _check(lib, lib.pae_paged_attention_decode(
        _ptr(out), _ptr(qkv), _ptr(keys), _ptr(values), _ptr(block_table), block_table.shape[1],
        _ptr(q_start), _ptr(kv_len), seqs, num_heads, num_kv_heads, head_dim,
        page_size, scale, window, slice_keys, max_slices,
        _ptr(scratch), _stream()), launches)


def paged_attention(qkv, keys, values, block_table, q_start, q_pos0, kv_len, num_heads, num_kv_heads, head_dim,
                    page_size, max_q_len, max_kv_len, scale, window, num_single=None, form: int = 0,
                    info: dict | None = None, multi_index: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of every token of the step over its request's pages. `num_single` is the number
    of requests that bring exactly one token when the caller knows it (it decides which kernels
    are launched; None launches whatever may be needed). `multi_index` (int32, device) lists the
    requests that bring more than one token when some do and some do not: the portion kernels
    then launch blocks for those only (a step of 64 decoding requests and one prompt portion
    otherwise launches 65 requests' worth of blocks, 64 of which return at once but not for free). `form` 0 lets the tcgen05 attention pick
    its kernel by the size of the launch (two blocks of 64-key tiles per SM when there are that
    many blocks, else one block of 128-key tiles, its keys shared out over a cluster when the
    blocks are few); 1, 2, 4, 8, 16 name the kernel (tests). `info`, when given, receives which
    kernel ran ("kernel") and, for tcgen05, the blocks per query tile ("cluster": 0 is the
    paired kernel)."""
    qkv = materialized(qkv)
    _need(qkv, "paged_attention: qkv")
    _need(keys, "paged_attention: keys", qkv.dtype)
    _need(values, "paged_attention: values", qkv.dtype)
    for name, t in (("block_table", block_table), ("q_start", q_start), ("q_pos0", q_pos0), ("kv_len", kv_len)):
        _need(t, f"paged_attention: {name}", torch.int32)
    tokens = qkv.shape[0]
    seqs = kv_len.numel()
    out = torch.empty((tokens, num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    if qkv.dtype == torch.bfloat16 and use_tensor_cores:
        lib = _lib("attention_mma")
        mma_ok = bool(lib.pae_attention_mma_supports(num_heads, num_kv_heads, head_dim, page_size))
        singles = num_single if num_single is not None else (seqs if max_q_len == 1 else -1)
        # The requests that bring more than one token, when the caller lists them and the decode kernel takes the others.
        listed = multi_index if (multi_index is not None and mma_ok and singles > 0) else None
        if listed is not None:
            _need(listed, "paged_attention: multi_index", torch.int32)
            if listed.numel() != seqs - singles:
                raise KernelError(f"paged_attention: {listed.numel()} requests listed, {seqs - singles} bring more than one token")
        # Portions of 64 tokens and more: both products on tcgen05, one thread per query row.
        if use_tcgen05_attention and max_q_len >= TCGEN05_ATTENTION_MIN_TOKENS:
            tc5 = _lib("attention_tcgen05")
            if tc5.pae_attention_tcgen05_supports(num_heads, num_kv_heads, head_dim, page_size):
                decode_after = mma_ok and singles != 0
                chosen = c_int(-1)
                _set_bounds("attention_tcgen05", keys)
                _check(tc5, tc5.pae_paged_attention_prefill_tcgen05(
                    _ptr(out), _ptr(qkv), _ptr(keys), _ptr(values), ctypes.c_longlong(keys.shape[0]), _ptr(block_table),
                    block_table.shape[1], _ptr(q_start), _ptr(q_pos0), _ptr(kv_len), tokens, seqs,
                    max_q_len, max_kv_len, num_heads, num_kv_heads, head_dim, page_size,
                    scale, window, (1 if decode_after else 0), singles, form,
                    ctypes.byref(chosen), _ptr(listed), (listed.numel() if listed is not None else 0),
                    _ptr(_error_flag(qkv.device)), _stream()))
                if info is not None:
                    info.update(kernel="tcgen05", cluster=chosen.value)
                if decode_after:
                    _decode_attention(lib, out, qkv, keys, values, block_table, q_start, kv_len, seqs, singles,
                                      num_heads, num_kv_heads, head_dim, page_size, max_kv_len, scale, window)
                return out
        if mma_ok:
            if info is not None:
                info.update(kernel="mma")
            if max_q_len > 1:
                _set_bounds("attention_mma", keys)
                _check(lib, lib.pae_paged_attention_prefill(
                    _ptr(out), _ptr(qkv), _ptr(keys), _ptr(values), _ptr(block_table), block_table.shape[1],
                    _ptr(q_start), _ptr(q_pos0), _ptr(kv_len), seqs, max_q_len, num_heads,
                    num_kv_heads, head_dim, page_size, scale, window,
                    1, _ptr(listed), (listed.numel() if listed is not None else 0), _stream()))
            if singles != 0:
                _decode_attention(lib, out, qkv, keys, values, block_table, q_start, kv_len, seqs, singles, num_heads,
                                  num_kv_heads, head_dim, page_size, max_kv_len, scale, window)
            return out
    if info is not None:
        info.update(kernel="simt")
    lib = _lib("attention_simt")
    _set_bounds("attention_simt", keys)
    _check(lib, lib.pae_paged_attention_simt(
        _ptr(out), _ptr(qkv), _ptr(keys), _ptr(values), _ptr(block_table), block_table.shape[1], _ptr(q_start),
        _ptr(q_pos0), _ptr(kv_len), seqs, max_q_len, num_heads, num_kv_heads,
        head_dim, page_size, scale, window, (_code(qkv)), _stream()))
    return out


def silu_mul(gate_up, block: int = 0) -> torch.Tensor:
    """silu(gate) * up of a [tokens, 2 I] product. block 0: gate is columns [0, I) and up [I, 2 I);
    block b: b gate columns, then their b up columns, and so on (`linear_swiglu`'s weight layout)."""
    tokens, two_i = gate_up.shape
    if two_i % 2 or (block and two_i % (2 * block)):
        raise KernelError(f"silu_mul: rows of {two_i} do not split into gate and up (blocks of {block})")
    if isinstance(gate_up, PendingSum) and gate_up.value is None and gate_up.bias is None and gate_up.residual is None:
        splits = gate_up.partial.shape[0]
        out = torch.empty((tokens, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
        lib = _lib("fused_decode")
        _check(lib, lib.pae_splitk_silu_mul(_ptr(out), _ptr(gate_up.partial), splits, tokens,
                                            (two_i // 2), block, _DTYPE_CODE[gate_up.dtype], _stream()))
        return out
    gate_up = materialized(gate_up)
    _need(gate_up, "silu_mul: gate_up")
    out = torch.empty((tokens, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    lib = _lib("elementwise")
    _check(lib, lib.pae_silu_mul(_ptr(out), _ptr(gate_up), tokens, (two_i // 2), block,
                                 (_code(gate_up)), _stream()))
    return out


SWIGLU_BLOCK = 16


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor | None:
    """[2 I, K] with 16 gate rows, their 16 up rows, and so on: the weight layout of
    `linear_swiglu`, in which a product's tile holds gate and up of the same columns. None
    when I is not a multiple of 16."""
    inter, k = gate.shape
    if inter % SWIGLU_BLOCK:
        return None
    both = torch.stack((gate.view(inter // SWIGLU_BLOCK, SWIGLU_BLOCK, k), up.view(inter // SWIGLU_BLOCK, SWIGLU_BLOCK, k)), dim=1)
    return both.reshape(2 * inter, k).contiguous()


def linear_swiglu(x, weight) -> torch.Tensor:
    """silu(x . Wg^T) * (x . Wu^T) -> [M, I] for a weight from `interleave_gate_up`. With many
    tokens the activation runs in the product's epilogue; with few, in the kernel that sums the
    splits; otherwise as a kernel of its own. Gate and up are rounded to the engine dtype first in
    every one of them, so all give the same bits."""
    source, norm_weight, eps = _norm_of(x)
    if (_few_tokens(source, weight.shape[1], norm_weight is not None, GATE_UP_KIND, weight.shape[0]) and weight.dtype == torch.bfloat16 and weight.is_contiguous()
            and weight.data_ptr() % 16 == 0 and weight.shape[0] % 32 == 0 and source.shape[1] == weight.shape[1]):
        _need(source, "linear_swiglu: x")
        out = torch.empty((source.shape[0], weight.shape[0] // 2), dtype=torch.bfloat16, device=source.device)
        lib = _lib("gemv_mma")
        _check(lib, lib.pae_linear_swiglu_few_tokens(_ptr(out), _ptr(source), _ptr(weight), _ptr(norm_weight), eps,
                                                     source.shape[0], weight.shape[0], weight.shape[1],
                                                     _ptr(_error_flag(source.device)), _stream()))
        return out
    x = materialized(x)
    m, k = x.shape
    n = weight.shape[0]
    if (m > SWIGLU_SWAPPED_MAX_TOKENS and n >= 256 and n % 32 == 0 and _tensor_core_shape(x, weight, None, x.dtype)
            and weight.shape[1] == k):
        _need(x, "linear_swiglu: x")
        _need(weight, "linear_swiglu: weight")
        out = torch.empty((m, n // 2), dtype=x.dtype, device=x.device)
        lib = _lib("gemm_tcgen05")
        _check(lib, lib.pae_linear_swiglu_tcgen05(_ptr(out), _ptr(x), _ptr(weight), m, n, k,
                                                  _ptr(_error_flag(x.device)), _stream()))
        return out
    return silu_mul(linear(x, weight), SWIGLU_BLOCK)


def sample(logits, temperature, seed_lo, seed_hi, request_key, output_index, keep=None) -> torch.Tensor:
    """int32 [rows]: argmax where temperature is 0, else the Gumbel-max draw of the row's counters.
    `keep` = (last_token, logit_rows, seq_index, state_slot): the kernel that picks a row's token
    also does what `scatter_tokens` would (one launch fewer in a step)."""
    _need(logits, "sample: logits", torch.float32)
    _need(temperature, "sample: temperature", torch.float32)
    for name, t in (("seed_lo", seed_lo), ("seed_hi", seed_hi), ("request_key", request_key), ("output_index", output_index)):
        _need(t, f"sample: {name}", torch.int32)
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    lib = _lib("sampling")
    words = lib.pae_sample_scratch_words(rows, vocab)
    scratch = torch.empty(words, dtype=torch.int32, device=logits.device) if words else None
    kept = (None, None, None, None)
    if keep is not None:
        kept = keep
        for name, t in zip(("last_token", "logit_rows", "seq_index", "state_slot"), kept):
            _need(t, f"sample: {name}", torch.int32)
        if kept[1].numel() != rows:
            raise KernelError(f"sample: {rows} rows of logits, {kept[1].numel()} wanted places")
    _check(lib, lib.pae_sample(_ptr(out), _ptr(logits), _ptr(temperature), _ptr(seed_lo), _ptr(seed_hi),
                               _ptr(request_key), _ptr(output_index), rows, vocab, _ptr(scratch),
                               _ptr(kept[0]), _ptr(kept[1]), _ptr(kept[2]), _ptr(kept[3]),
                               _stream()), 2 if words else 1)
    return out
