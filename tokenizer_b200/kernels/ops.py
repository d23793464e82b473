"""Python faces of the CUDA launchers.  Every function takes CUDA tensors,
launches on the current stream and raises instead of returning a wrong result:
`KernelError` for a launch that failed, `ValueError` for a size a kernel
refuses.  There is no CPU path: a tensor that is not on a GPU is an error."""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .build import load_library

F32, BF16 = 0, 1
_DTYPE_TAG = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


_STATUS_TEXT = {
    -1: "a size this kernel does not take",
    -2: "a dtype this kernel does not take",
    -3: "a pointer or stride that is not aligned as the kernel needs",
    -4: "a bounded wait on the device ran out",
}


class _Counter:
    """How many of the framework's own kernels were launched (the bench reports it)."""
    launches = 0


counter = _Counter()


def _check(status: int, what: str) -> None:
    if status == 0:
        counter.launches += 1
        return
    if status < 0:
        raise ValueError(f"{what}: {_STATUS_TEXT.get(status, f'status {status}')}")
    raise KernelError(f"{what}: CUDA error {status} at launch")


def _tag(t: torch.Tensor) -> int:
    try:
        return _DTYPE_TAG[t.dtype]
    except KeyError:
        raise ValueError(f"kernels take float32 or bfloat16, found {t.dtype}") from None


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise KernelError("tokenizer_b200 kernels run on a GPU only; got a CPU tensor")
    if not t.is_contiguous():
        raise ValueError("kernels take contiguous tensors")
    return ctypes.c_void_p(t.data_ptr())


_bound_stream = None


def _stream():
    if _bound_stream is not None:
        return _bound_stream
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class bound_stream:
    """Within the block every launch goes to the stream that is current at its entry, looked
    up once (asking torch for the current stream costs several microseconds, and a step has a
    few hundred launches).  Nest it anew where the current stream changes (a second stream, a
    graph capture)."""

    def __enter__(self):
        global _bound_stream
        self._outer = _bound_stream
        _bound_stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        global _bound_stream
        _bound_stream = self._outer
        return False


_i, _f, _ll = ctypes.c_int, ctypes.c_float, ctypes.c_longlong


class ScratchSpace:
    """Device memory that kernels use beyond their inputs and outputs: the pieces and counters
    of the decode attention, the activation and barrier counters of the fused feed-forward,
    the partial results of the greedy choice.  Counters are zero between launches, and two
    launches that overlap on the device must not share them, so a space belongs to ONE order
    of launches: a model (its forward runs on one stream) and a sampler each own theirs
    (`scratch_scope`), and die with them.  Launches outside any scope (kernel tests) share
    the module's default space, on one stream.  Buffers are made at a shape's first use,
    which is never inside a captured graph: a shape's first step runs plainly."""

    def __init__(self):
        self.decode, self.ffn, self.argmax, self.layer = {}, {}, {}, {}


_default_space = ScratchSpace()
_space = _default_space


class scratch_scope:
    """Within the block, kernels take their scratch from `space`."""

    def __init__(self, space: ScratchSpace):
        self.space = space

    def __enter__(self):
        global _space
        self._outer = _space
        _space = self.space
        return self

    def __exit__(self, *exc):
        global _space
        _space = self._outer
        return False


# ---- the error word ----------------------------------------------------------------
# A wait on the device that runs out does not hang: the kernel sets its library's flag, stores a
# code in one word of mapped pinned host memory and runs to its end WITHOUT the data it waited
# for, so what it wrote is wrong.  Every library gets the word's device address when it is
# loaded; the host reads the word (plain memory, no CUDA call) wherever it has just
# synchronised with the device, and raises.
_LIBRARY_NAMES = {1: "gemm_tcgen05", 2: "attention_tcgen05", 3: "ffn_small_m", 4: "linear_stream",
                  5: "layer_small_m"}
_REASONS = {1: "a wait on a shared-memory barrier ran out", 2: "a wait between blocks ran out"}
_error_word = None          # (ctypes int at the host address, device address)
_registered = {}            # id(library handle) -> handle: libraries that know the word


def _error_word_pointers():
    global _error_word
    if _error_word is None:
        lib = load_library("elementwise.cu")
        host, dev = ctypes.c_void_p(0), ctypes.c_void_p(0)
        status = lib.tokb200_error_word_alloc(ctypes.byref(host), ctypes.byref(dev))
        if status != 0 or not host.value:
            raise KernelError(f"the error word could not be allocated (CUDA error {status})")
        _error_word = (ctypes.c_int.from_address(host.value), dev.value)
    return _error_word


def _load(source: str, defines=()):
    """Load (compile at first use) a library and hand it the error word."""
    lib = load_library(source, defines=defines)
    if id(lib) not in _registered:
        _, dev = _error_word_pointers()
        status = lib.tokb200_set_error_word(ctypes.c_void_p(dev))
        if status != 0:
            raise KernelError(f"{source}: the error word could not be set (CUDA error {status})")
        _registered[id(lib)] = lib
    return lib


def _lib(name):
    return _load(name + ".cu")


def error_code() -> int:
    """The word as it stands (0: no bounded wait has run out); meaningful once the device has
    finished the work in question."""
    return 0 if _error_word is None else int(_error_word[0].value)


def raise_if_error(where: str = "") -> None:
    """Raise KernelError if a bounded wait on the device ran out since the last check.  The
    word and the libraries' flags are cleared, so the next step starts clean.  Costs a read of
    host memory when nothing happened; call it after a synchronisation with the device."""
    code = error_code()
    if code == 0:
        return
    _error_word[0].value = 0
    library, reason = _LIBRARY_NAMES.get(code // 16, f"library {code // 16}"), code % 16
    if reason == 2 and code // 16 == 2:
        text = "a shared-memory base was not aligned as the kernel needs"
    else:
        text = _REASONS.get(reason, f"reason {reason}")
    for lib in _registered.values():          # clear the per-library flags too
        for name in ("tokb200_gemm_tcgen05_error", "tokb200_attention_tcgen05_error",
                     "tokb200_ffn_small_m_error", "tokb200_linear_stream_error",
                     "tokb200_layer_small_m_error"):
            try:
                getattr(lib, name)()
            except AttributeError:
                pass
    raise KernelError(f"{library}: {text}{' (' + where + ')' if where else ''}; the results of the "
                      f"steps since the last check are not valid")


# --------------------------------------------------------------------------- #
def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    n, hidden = out.shape
    _check(_lib("elementwise").tokb200_embed(
        _ptr(ids), _ptr(table), _i(_tag(table)), _ptr(out), _i(n), _i(hidden),
        _i(table.shape[0]), _stream()), "embed")


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor,
             delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> None:
    """out = norm(x [+ delta]) * gain; with `delta`, x is updated in place.  With
    `rows` (int32), only those rows are read and `out` is dense [len(rows), H]."""
    hidden = x.shape[-1]
    n_rows = out.shape[0]
    if x.dtype != torch.float32 or gain.dtype != torch.float32:
        raise ValueError("rms_norm: the residual stream and the gain are float32")
    if gain.numel() != hidden or out.shape[-1] != hidden:
        raise ValueError("rms_norm: sizes of x, gain and out disagree")
    if delta is not None and rows is not None:
        raise ValueError("rms_norm: a pending residual and a row gather do not combine")
    n_partials, stride = _partials(delta, x)
    _check(_lib("elementwise").tokb200_rms_norm(
        _ptr(x), _ptr(delta), _i(_tag(delta) if delta is not None else F32), _i(n_partials),
        _ll(stride), _ptr(gain),
        _ptr(out), _i(_tag(out)), _ptr(rows), _i(n_rows), _i(hidden), _f(eps), _stream()),
        "rms_norm")


def _partials(delta, x):
    """A pending residual is [T, H], or float32 partial sums [S, T, H] of a
    product that was cut along k; returns (S, elements between partials)."""
    if delta is None or delta.dim() == x.dim():
        if delta is not None and delta.shape != x.shape:
            raise ValueError("the pending residual has another shape than the stream")
        return 1, 0
    if delta.dim() != x.dim() + 1 or delta.shape[1:] != x.shape or delta.dtype != torch.float32:
        raise ValueError("partial sums are float32 [S, T, H]")
    return delta.shape[0], x.numel()


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> None:
    if x.dtype != torch.float32:
        raise ValueError("residual_add: x is float32")
    n_partials, _ = _partials(delta, x)
    _check(_lib("elementwise").tokb200_residual_add(
        _ptr(x), _ptr(delta), _i(_tag(delta)), _i(n_partials), _ll(x.numel()), _stream()),
        "residual_add")


def rope_table(inv_freq: torch.Tensor, n_positions: int):
    half = inv_freq.numel()
    cos = torch.empty((n_positions, half), dtype=torch.float32, device=inv_freq.device)
    sin = torch.empty_like(cos)
    _check(_lib("elementwise").tokb200_rope_table(
        _ptr(inv_freq), _ptr(cos), _ptr(sin), _i(n_positions), _i(half), _stream()), "rope_table")
    return cos, sin


def rope_store(qkv, bias, pos, slot, cos, sin, q_out, k_pool, v_pool, nh, nkv, d, rotary) -> None:
    """Bias, rotation and the write of k and v to their cache slots.  `qkv` is [T, width] or
    float32 partial sums [S, T, width] of a product cut along k (bfloat16 outputs, the whole
    head rotated, head size a multiple of 16)."""
    if qkv.dim() == 3:
        n = qkv.shape[1]
        if qkv.dtype != torch.float32 or qkv.shape[2] != (nh + 2 * nkv) * d or rotary != d or d % 16 or \
                q_out.dtype != torch.bfloat16 or cos.shape[1] != d // 2:
            raise ValueError("rope_store: partial sums are float32 [S, T, width], for bfloat16 "
                             "outputs and a whole-head rotation with head size a multiple of 16")
        _check(_lib("elementwise").tokb200_rope_store_partials(
            _ptr(qkv), _i(qkv.shape[0]), _ptr(bias), _ptr(pos), _ptr(slot), _ptr(cos), _ptr(sin),
            _ptr(q_out), _ptr(k_pool), _ptr(v_pool), _i(n), _i(nh), _i(nkv), _i(d), _stream()),
            "rope_store_partials")
        return
    n = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * d:
        raise ValueError("rope_store: qkv width is not (heads + 2 kv heads) * head_dim")
    if rotary % 2 or (d - rotary) % 2 or rotary > d or cos.shape[1] != rotary // 2:
        raise ValueError(f"rope_store: rotary width {rotary} does not fit head size {d}")
    _check(_lib("elementwise").tokb200_rope_store(
        _ptr(qkv), _ptr(bias), _ptr(pos), _ptr(slot), _ptr(cos), _ptr(sin), _ptr(q_out),
        _ptr(k_pool), _ptr(v_pool), _i(_tag(qkv)), _i(n), _i(nh), _i(nkv), _i(d), _i(rotary),
        _stream()), "rope_store")


# The activation of a gated feed-forward is a parameter of every kernel that applies one.
ACTIVATIONS = {"silu": 0, "gelu_pytorch_tanh": 1, "relu": 2}


def activation_tag(name: str) -> int:
    try:
        return ACTIVATIONS[name]
    except KeyError:
        raise ValueError(f"the gated kernels know the activations {', '.join(ACTIVATIONS)}; found {name!r}") from None


def silu_gate(gu: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """out[t, i] = act(gu[t, i]) * gu[t, I + i] (the name is from the activation of the
    architecture served; any of `ACTIVATIONS` is taken)."""
    n, inner = out.shape
    if gu.shape[1] != 2 * inner or gu.dtype != out.dtype:
        raise ValueError("silu_gate: input is [T, 2 I], output [T, I], same dtype")
    _check(_lib("elementwise").tokb200_silu_gate(
        _ptr(gu), _ptr(out), _i(_tag(gu)), _i(n), _i(inner), _i(activation_tag(activation)), _stream()),
        "silu_gate")


def paged_attention_generic(q, k_pool, v_pool, out, block_table, row_req, pos, nh, nkv, d, page,
                            window, scale) -> None:
    if d > 512:
        raise ValueError(f"attention: head size {d} is beyond 512")
    if nh % nkv:
        raise ValueError(f"attention: {nh} heads do not divide into {nkv} groups")
    _check(_lib("attention_generic").tokb200_paged_attention_generic(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _i(_tag(q)), _ptr(block_table),
        _i(block_table.shape[1]), _ptr(row_req), _ptr(pos), _i(q.shape[0]), _i(nh), _i(nkv),
        _i(d), _i(page), _i(-1 if window is None else int(window)), _f(scale), _stream()),
        "paged_attention")


def gemm_f32(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor],
             out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] w[N,K]^T (+ bias), true 32-bit."""
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise ValueError("gemm_f32: shapes do not chain")
    for t in (a, w, out):
        if t.dtype != torch.float32:
            raise ValueError("gemm_f32 takes float32")
    _check(_lib("gemm_f32").tokb200_gemm_f32(
        _ptr(a), _ptr(w), _ptr(bias), _ptr(out), _i(M), _i(N), _i(K), _i(K), _i(N), _stream()),
        "gemm_f32")


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor],
           top_p: Optional[torch.Tensor], uniform: Optional[torch.Tensor],
           out: torch.Tensor) -> None:
    """One token per row of float32 logits; all-None parameters mean greedy."""
    if logits.dtype != torch.float32 or out.dtype != torch.int32:
        raise ValueError("sample: logits are float32, ids int32")
    if temperature is None:
        return argmax(logits, out)
    _check(_lib("sampling").tokb200_sample(
        _ptr(logits), _i(logits.shape[0]), _i(logits.shape[1]), _ptr(temperature), _ptr(top_p),
        _ptr(uniform), _ptr(out), _stream()), "sample")


def prefetch_l2(t: torch.Tensor) -> None:
    """Ask for a tensor's bytes to be brought into L2; returns at once."""
    _check(_lib("elementwise").tokb200_prefetch_l2(
        _ptr(t), _ll(t.numel() * t.element_size()), _stream()), "prefetch_l2")


def advance_decode(ids, drawn, pos, kv_len, row_req, slots, tables, page, history,
                   step_counter) -> None:
    """After a decoding step: the drawn ids become the next inputs and every
    row's position, stored length and cache slot move on by one (on the device)."""
    n = len(slots)
    if n > 4:
        raise ValueError("advance_decode handles up to four cache groups")
    slot_ptrs = (ctypes.c_void_p * max(n, 1))(*[t.data_ptr() for t in slots])
    table_ptrs = (ctypes.c_void_p * max(n, 1))(*[t.data_ptr() for t in tables])
    widths = (ctypes.c_int * max(n, 1))(*[t.shape[1] for t in tables])
    _check(_lib("elementwise").tokb200_advance_decode(
        _ptr(ids), _ptr(drawn), _ptr(pos), _ptr(kv_len), _ptr(row_req), _i(n), slot_ptrs,
        table_ptrs, widths, _i(page), _i(ids.shape[0]), _ptr(history), _ptr(step_counter),
        _stream()), "advance_decode")


DECODE_MAX_GROUP = 16


def decode_attention_supported(nh: int, nkv: int, d: int) -> bool:
    """Sizes the split-key decoding kernel takes; others go to the general kernel."""
    return d % 16 == 0 and 16 <= d <= 256 and nh % nkv == 0 and nh // nkv <= DECODE_MAX_GROUP


def decode_attention(q, k_pool, v_pool, out, block_table, row_req, pos, nh, nkv, d, page, window,
                     scale, rows: Optional[torch.Tensor] = None) -> None:
    """Attention for rows of one token each (bfloat16): keys are split over
    blocks and merged; the scratch for the pieces is kept per (device, rows,
    heads, head size) and reused by every layer, which run one after another.  With `rows`
    (int32, -1 for none) only those rows of the batch are served: the single-token rows of a
    step that also brings portions of prompts, which go to the kernels for portions."""
    if q.dtype != torch.bfloat16:
        raise ValueError("decode_attention is the bfloat16 kernel")
    if not decode_attention_supported(nh, nkv, d):
        raise ValueError(f"decode_attention: {nh} heads over {nkv} groups of size {d} is not taken")
    lib = _load("attention_decode.cu", defines=(f"HEAD_DIM={d}",))
    n_rows = q.shape[0] if rows is None else rows.shape[0]
    key = (q.device.index, n_rows, nh, nkv, d)
    if key not in _space.decode:
        lib.tokb200_decode_attention_scratch_floats.restype = ctypes.c_longlong
        floats = lib.tokb200_decode_attention_scratch_floats(_i(n_rows), _i(nh))
        _space.decode[key] = (torch.empty(floats, dtype=torch.float32, device=q.device),
                              torch.zeros(n_rows * nkv, dtype=torch.int32, device=q.device))
    scratch, counters = _space.decode[key]
    _check(lib.tokb200_decode_attention(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(block_table),
        _i(block_table.shape[1]), _ptr(row_req), _ptr(pos), _i(n_rows), _i(nh), _i(nkv), _i(d),
        _i(page), _i(-1 if window is None else int(window)), _f(scale), _ptr(scratch),
        _ptr(counters), _ptr(rows), _stream()), "decode_attention")


_stream_plans = {}


def linear_stream_supported(M: int, N: int, K: int) -> bool:
    """Sizes the ring-streaming product takes on this device (up to 16 rows, K a multiple of
    32 up to 8192); it pays for matrices of many rows (several tiles of 16 per SM)."""
    if M < 1 or M > 16 or K % 32 or K > 8192:
        return False
    key = (torch.cuda.current_device(), M <= 8, N, K)
    if key not in _stream_plans:
        _stream_plans[key] = bool(_lib("linear_stream").tokb200_linear_stream_supported(_i(M), _i(N), _i(K)))
    return _stream_plans[key]


def linear_stream(x, w, bias, out) -> None:
    """out[M,N] = x w^T (+ bias float32) for up to 16 rows of bfloat16 x and a weight of many
    rows, streamed through shared memory by bulk copies; out is bfloat16 or float32."""
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise ValueError("linear_stream: bfloat16 x [M,K] and w [N,K]")
    if tuple(out.shape) != (M, N) or out.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("linear_stream: out is [M,N] bfloat16 or float32")
    if not linear_stream_supported(M, N, K):
        raise ValueError(f"linear_stream does not take {M} rows with K = {K}")
    _check(_lib("linear_stream").tokb200_linear_stream(
        _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _i(1 if out.dtype == torch.float32 else 0),
        _i(M), _i(N), _i(K), _stream()), "linear_stream")


def linear_stream_check() -> None:
    flag = _lib("linear_stream").tokb200_linear_stream_error()
    if flag:
        raise KernelError("linear_stream: a wait on the device ran out (status %d)" % flag)


_ffn_plans = {}
# compile-time switches of the fused feed-forward's library (a test builds it with short wait limits)
_FFN_DEFINES = ()


def _ffn_lib():
    return _load("ffn_small_m.cu", defines=_FFN_DEFINES)


def ffn_small_m_splits(M: int, hidden: int, inner: int) -> int:
    """Partial sums the fused feed-forward of few rows writes for these sizes on this
    device; 0 when it does not take them (more than 16 rows, hidden not a multiple of
    32, inner not a multiple of 128, too little shared memory)."""
    key = (torch.cuda.current_device(), M <= 8, hidden, inner)
    if M < 1 or M > 16:
        return 0
    if key not in _ffn_plans:
        _ffn_plans[key] = int(_ffn_lib().tokb200_ffn_small_m_splits(_i(M), _i(hidden), _i(inner)))
    return _ffn_plans[key]


def ffn_small_m(x_in, x_out, delta, gain, eps, w_gate_up, w_down, out, activation: str = "silu") -> None:
    """The gated feed-forward of few rows in one kernel: x_out = x_in + delta (delta as
    for rms_norm: [M, H] or float32 partial sums [S, M, H], or None), out [S', M, H] =
    float32 partial sums over k of down(act(gate(h)) * up(h)), h = rms_norm(x_out) * gain.
    `w_gate_up` is in the interleaved row order of `interleave_gate_up`."""
    M, hidden = x_in.shape
    inner = w_down.shape[1]
    if x_in.dtype != torch.float32 or x_out.dtype != torch.float32 or x_out.shape != x_in.shape:
        raise ValueError("ffn_small_m: the residual stream is float32, in and out of one shape")
    if w_gate_up.dtype != torch.bfloat16 or w_down.dtype != torch.bfloat16 or \
            tuple(w_gate_up.shape) != (2 * inner, hidden) or tuple(w_down.shape) != (hidden, inner):
        raise ValueError("ffn_small_m: bfloat16 weights [2 I, H] and [H, I]")
    splits = ffn_small_m_splits(M, hidden, inner)
    if splits == 0:
        raise ValueError(f"ffn_small_m does not take {M} rows of {hidden} with inner size {inner}")
    if tuple(out.shape) != (splits, M, hidden) or out.dtype != torch.float32:
        raise ValueError(f"ffn_small_m: out must be float32 {(splits, M, hidden)}")
    n_partials, stride = _partials(delta, x_in)
    key = (x_in.device.index, inner)
    if key not in _space.ffn:
        _space.ffn[key] = (torch.empty((16, inner), dtype=torch.bfloat16, device=x_in.device),
                           torch.zeros(2, dtype=torch.int32, device=x_in.device))
    act, sync = _space.ffn[key]
    _check(_ffn_lib().tokb200_ffn_small_m(
        _ptr(x_in), _ptr(x_out), _ptr(delta), _i(1 if delta is not None and delta.dtype == torch.float32 else 0),
        _i(n_partials), _ll(stride), _ptr(gain), _f(eps), _ptr(w_gate_up), _ptr(w_down), _ptr(act),
        _ptr(out), _i(M), _i(hidden), _i(inner), _i(activation_tag(activation)), _ptr(sync), _stream()),
        "ffn_small_m")


def ffn_small_m_check() -> None:
    flag = _ffn_lib().tokb200_ffn_small_m_error()
    if flag:
        raise KernelError("ffn_small_m: a wait on the device ran out (status %d)" % flag)


SMALL_M_ROWS = 16     # up to here the streaming kernel leads; above it, the tensor-core tiles


def linear_small_m_supported(M: int, K: int) -> bool:
    return 0 < M <= 64 and K % 8 == 0


def linear_small_m(x, w, bias, out, k_splits: int = 1) -> None:
    """out = x w^T (+ bias) for at most 64 rows of bfloat16 x.  With k_splits > 1
    `out` is float32 [k_splits, M, N]: partial sums that the consumer adds."""
    M, K = x.shape
    N = w.shape[0]
    if not linear_small_m_supported(M, K):
        raise ValueError(f"linear_small_m takes up to 64 rows and K a multiple of 8; got {M} x {K}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise ValueError("linear_small_m: bfloat16 x [M,K] and w [N,K]")
    want = (M, N) if k_splits == 1 else (k_splits, M, N)
    if tuple(out.shape) != want or (k_splits > 1 and out.dtype != torch.float32):
        raise ValueError(f"linear_small_m: out must be {want}")
    _check(_lib("linear_small_m").tokb200_linear_small_m(
        _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _i(1 if out.dtype == torch.float32 else 0),
        _i(M), _i(N), _i(K), _i(k_splits), _stream()), "linear_small_m")


PREFILL_TILE_ROWS = 64


def prefill_attention_supported(nh: int, nkv: int, d: int) -> bool:
    return d % 16 == 0 and 16 <= d <= 128 and nh % nkv == 0


def prefill_attention(q, k_pool, v_pool, out, block_table, row_req, pos, tiles, n_tiles, nh, nkv,
                      d, page, window, scale) -> None:
    """Attention for portions of prompts (bfloat16).  `tiles` is int32 [n, 2]:
    (first row, rows <= 64) of consecutive rows of one request."""
    if q.dtype != torch.bfloat16:
        raise ValueError("prefill_attention is the bfloat16 kernel")
    if not prefill_attention_supported(nh, nkv, d):
        raise ValueError(f"prefill_attention: {nh} heads over {nkv} groups of size {d} is not taken")
    lib = _load("attention_prefill.cu", defines=(f"HEAD_DIM={d}",))
    _check(lib.tokb200_prefill_attention(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(block_table),
        _i(block_table.shape[1]), _ptr(row_req), _ptr(pos), _ptr(tiles), _i(n_tiles), _i(nh),
        _i(nkv), _i(d), _i(page), _i(-1 if window is None else int(window)), _f(scale), _stream()),
        "prefill_attention")


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """Greedy ids (ties keep the lower id): the vocabulary is cut over blocks
    that meet in scratch kept per (device, rows)."""
    n_rows, vocab = logits.shape
    lib = _lib("sampling")
    key = (logits.device.index, n_rows)
    if key not in _space.argmax:
        lib.tokb200_argmax_scratch_bytes.restype = ctypes.c_longlong
        size = lib.tokb200_argmax_scratch_bytes(_i(n_rows))
        _space.argmax[key] = (torch.empty(size, dtype=torch.uint8, device=logits.device),
                              torch.zeros(n_rows, dtype=torch.int32, device=logits.device))
    scratch, counters = _space.argmax[key]
    _check(lib.tokb200_argmax(_ptr(logits), _i(n_rows), _i(vocab), _ptr(out), _ptr(scratch),
                              _ptr(counters), _stream()), "argmax")


def gemm_tcgen05_supported(M: int, N: int, K: int) -> bool:
    return M > 0 and N > 0 and K > 0 and K % 8 == 0


def gemm_tcgen05(a, w, bias, out, block_n: int = 0) -> None:
    """out[M,N] = a[M,K] w[N,K]^T (+ bias) on tcgen05 tensor cores with TMA-fed
    operands; bfloat16 in, bfloat16 or float32 out.  K must be a multiple of 8."""
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise ValueError("gemm_tcgen05: bfloat16 a [M,K] and w [N,K]")
    if not gemm_tcgen05_supported(M, N, K):
        raise ValueError(f"gemm_tcgen05: K = {K} must be a multiple of 8")
    if tuple(out.shape) != (M, N) or out.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("gemm_tcgen05: out is [M,N] bfloat16 or float32")
    if not block_n:
        pitch_ok = N % (4 if out.dtype == torch.float32 else 8) == 0
        if pitch_ok and M * N >= 128 * 128 * 32:
            # persistent kernel, TMA-stored output: the wide tile where it divides the work well
            # (with one tile of rows, the narrow tile gives twice the blocks to stream the weights)
            block_n = 1256 if (out.dtype == torch.bfloat16 and N >= 2048 and M > 128) else 1128
        else:
            block_n = 128 if N > 64 else 64
    _check(_lib("gemm_tcgen05").tokb200_gemm_tcgen05(
        _ptr(a), _ptr(w), _ptr(bias), _ptr(out), _i(1 if out.dtype == torch.float32 else 0),
        _i(M), _i(N), _i(K), _i(block_n), _stream()), "gemm_tcgen05")


def gemm_tcgen05_partials(a, w, out) -> None:
    """out[S,M,N] (float32) = partial sums of a[M,K] w[N,K]^T over S pieces of k, for products
    with too few output tiles to fill the device; the consumer adds the pieces in index order."""
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise ValueError("gemm_tcgen05_partials: bfloat16 a [M,K] and w [N,K]")
    if out.dim() != 3 or tuple(out.shape[1:]) != (M, N) or out.dtype != torch.float32:
        raise ValueError("gemm_tcgen05_partials: out is float32 [S,M,N]")
    if K % 8 or N % 4:
        raise ValueError("gemm_tcgen05_partials: K a multiple of 8 and N a multiple of 4")
    _check(_lib("gemm_tcgen05").tokb200_gemm_tcgen05_partials(
        _ptr(a), _ptr(w), _ptr(out), _i(M), _i(N), _i(K), _i(out.shape[0]), _stream()),
        "gemm_tcgen05_partials")


PAIR_PLAIN, PAIR_GATED, PAIR_PARTIALS, PAIR_PLAIN_128 = 0, 1, 2, 3
# TOKB200_GEMM_PAIR=0 keeps every tensor-core product on lone CTAs
_PAIR = os.environ.get("TOKB200_GEMM_PAIR", "1") != "0"


def gemm_tcgen05_pair(a, w, bias, out, kind: int, activation: str = "silu") -> None:
    """The product on pairs of CTAs (two SMs a tile of 256 rows x 256 columns, each loading half
    of the tile's rows of w).  PAIR_PLAIN: out [M,N] bfloat16 (+ bias); PAIR_GATED: out [M,N/2]
    bfloat16 = silu(gate) * up for w from `interleave_gate_up`; PAIR_PARTIALS: out [S,M,N]
    float32 partial sums over S pieces of k; PAIR_PLAIN_128: as PAIR_PLAIN with 128-column tiles."""
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise ValueError("gemm_tcgen05_pair: bfloat16 a [M,K] and w [N,K]")
    splits = 1
    if kind == PAIR_PARTIALS:
        if out.dim() != 3 or tuple(out.shape[1:]) != (M, N) or out.dtype != torch.float32 or bias is not None:
            raise ValueError("gemm_tcgen05_pair: partial sums are float32 [S,M,N] without bias")
        splits = out.shape[0]
    elif kind == PAIR_GATED:
        if tuple(out.shape) != (M, N // 2) or out.dtype != torch.bfloat16 or N % 256 or bias is not None:
            raise ValueError("gemm_tcgen05_pair: the gated product is bfloat16 [M,N/2], N a multiple of 256")
    elif kind in (PAIR_PLAIN, PAIR_PLAIN_128):
        if tuple(out.shape) != (M, N) or out.dtype != torch.bfloat16:
            raise ValueError("gemm_tcgen05_pair: out is bfloat16 [M,N]")
    else:
        raise ValueError(f"gemm_tcgen05_pair: kind {kind}")
    if K % 8 or N % (4 if kind == PAIR_PARTIALS else 8):
        raise ValueError("gemm_tcgen05_pair: K a multiple of 8, N of 8 (4 for partial sums)")
    _check(_lib("gemm_tcgen05").tokb200_gemm_tcgen05_pair(
        _ptr(a), _ptr(w), _ptr(bias), _ptr(out), _i(kind), _i(M), _i(N), _i(K), _i(splits),
        _i(activation_tag(activation)), _stream()), "gemm_tcgen05_pair")


def gemm_tcgen05_check() -> None:
    """Raise if a bounded wait inside the tensor-core product ran out since the last check."""
    flag = _lib("gemm_tcgen05").tokb200_gemm_tcgen05_error()
    if flag:
        raise KernelError("gemm_tcgen05: a wait on the device ran out (status %d)" % flag)


def gated_linear_supported(K: int, N: int) -> bool:
    """Gate and up products with the activation folded into the epilogue: the
    stacked weight is laid out in blocks of 128 gate rows + 128 up rows."""
    return K % 8 == 0 and N % 256 == 0


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[gate rows 0..127, up rows 0..127, gate rows 128..255, ...]: the layout the
    gated kernels read (both have I rows, I a multiple of 128)."""
    inner, k = gate.shape
    return torch.stack([gate.view(inner // 128, 128, k), up.view(inner // 128, 128, k)], dim=1) \
        .reshape(2 * inner, k).contiguous()


def gated_linear(x, w, out, activation: str = "silu") -> None:
    """out[M, N/2] = act(x Wg^T) * (x Wu^T) for w from `interleave_gate_up`; the activation
    is an epilogue parameter of whichever kernel the row count selects."""
    act = _i(activation_tag(activation))
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise ValueError("gated_linear is the bfloat16 kernel")
    if not gated_linear_supported(K, N) or w.shape[1] != K or tuple(out.shape) != (M, N // 2):
        raise ValueError("gated_linear: K a multiple of 8, N of 256, out [M, N/2]")
    if M <= SMALL_M_ROWS and _RING and N * K >= RING_ELEMENTS and linear_ring_supported(M, N, K, 1, True):
        linear_ring_gated(x, w, out, activation)
    elif M <= SMALL_M_ROWS:
        _check(_lib("linear_small_m").tokb200_linear_small_m_gated(
            _ptr(x), _ptr(w), _ptr(out), _i(M), _i(N), _i(K), act, _stream()), "gated_linear")
    elif M <= RING_MAX_ROWS and _RING and (M <= 24 or N * K <= 9_000_000) and linear_ring_supported(M, N, K, 1, True):
        # 17 to 32 rows: the ring kernel where it leads a tensor-core tile that is mostly padding
        # followed by the activation's own kernel (us in a captured chain, hidden 896: 11.3 -> 9.0
        # at 17 rows, 13.3 -> 10.6 at 32; hidden 1,536: 24.3 -> 17.5 at 17 rows, but 18.8 -> 20.6 at 32)
        linear_ring_gated(x, w, out, activation)
    elif M <= 64:
        # too few rows to fill the 256-wide gated tiles over the SMs: the plain tensor-core
        # product over the same (interleaved) weight, then the activation on its output
        gu = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        gemm_tcgen05(x, w, None, gu)
        _check(_lib("elementwise").tokb200_silu_gate_interleaved(
            _ptr(gu), _ptr(out), _i(M), _i(N // 2), act, _stream()), "silu_gate_interleaved")
    elif M >= 256 and _PAIR:
        # two tiles of rows and more: pairs of CTAs on tiles of 256 rows, each loading half of the
        # weight tile (a sixth fewer cycles than lone CTAs at 2,048 rows)
        _check(_lib("gemm_tcgen05").tokb200_gemm_tcgen05_pair(
            _ptr(x), _ptr(w), None, _ptr(out), _i(PAIR_GATED), _i(M), _i(N), _i(K), _i(1), act, _stream()),
            "gated_linear")
    else:
        _check(_lib("gemm_tcgen05").tokb200_gemm_tcgen05_gated(
            _ptr(x), _ptr(w), _ptr(out), _i(M), _i(N), _i(K), act, _stream()), "gated_linear")


def qkv_rope_small_m_supported(M: int, K: int, d: int, rotary: int, n_out: int = 0) -> bool:
    """Where the fused kernel is the one to use (it takes up to 64 rows).  Up to 32 rows: beyond 16 the streaming product is no longer the fastest on its own, but
    with rotation and cache write in its epilogue it still beats a tile product and a second
    kernel.  Up to 64 rows where the stacked weight is small (`n_out` x K up to two million
    elements: the 0.5B sizes), so that the product's own time hardly matters beside a launch
    saved (batch 64: 1.37 -> 1.28 ms a step)."""
    most = 64 if 0 < n_out * K <= 2_000_000 else 32
    return 0 < M <= most and K % 8 == 0 and d % 16 == 0 and rotary == d


def qkv_rope_small_m(x, w, bias, pos, slot, cos, sin, q_out, k_pool, v_pool, nh, nkv, d) -> None:
    """The stacked q/k/v projection of few rows with bias, rotary encoding and the
    cache write folded into its epilogue (bfloat16; the whole head is rotated)."""
    M, K = x.shape
    if w.shape != ((nh + 2 * nkv) * d, K) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise ValueError("qkv_rope_small_m: w is the stacked [(heads + 2 kv heads) d, K] weight")
    if not (0 < M <= 64 and K % 8 == 0 and d % 16 == 0 and 2 * cos.shape[1] == d):
        raise ValueError("qkv_rope_small_m: up to 64 rows, K a multiple of 8, the whole head (a multiple of 16) rotated")
    _check(_lib("linear_small_m").tokb200_qkv_rope_small_m(
        _ptr(x), _ptr(w), _ptr(bias), _ptr(pos), _ptr(slot), _ptr(cos), _ptr(sin), _ptr(q_out),
        _ptr(k_pool), _ptr(v_pool), _i(M), _i(nh), _i(nkv), _i(d), _i(K), _stream()),
        "qkv_rope_small_m")


def gemm_qkv_rope_supported(K: int, nh: int, nkv: int, d: int, rotary: int) -> bool:
    """Sizes the tcgen05 q/k/v product with the rotary epilogue takes: head size 64 or 128, the
    whole head rotated, and q and k/v regions of whole 128-column tiles."""
    return K % 8 == 0 and d in (64, 128) and rotary == d and (nh * d) % 128 == 0 and (nkv * d) % 128 == 0


def gemm_qkv_rope(x, w, bias, pos, slot, cos, sin, q_out, k_pool, v_pool, nh, nkv, d) -> None:
    """The stacked q/k/v projection of many rows on tcgen05 with bias, rotary encoding and the
    cache write folded into the epilogue (bfloat16)."""
    M, K = x.shape
    if w.shape != ((nh + 2 * nkv) * d, K) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise ValueError("gemm_qkv_rope: w is the stacked [(heads + 2 kv heads) d, K] weight")
    if not gemm_qkv_rope_supported(K, nh, nkv, d, 2 * cos.shape[1]) or tuple(q_out.shape) != (M, nh * d):
        raise ValueError("gemm_qkv_rope: sizes it does not take")
    _check(_lib("gemm_tcgen05").tokb200_gemm_tcgen05_qkv_rope(
        _ptr(x), _ptr(w), _ptr(bias), _ptr(pos), _ptr(slot), _ptr(cos), _ptr(sin), _ptr(q_out),
        _ptr(k_pool), _ptr(v_pool), _i(M), _i(nh), _i(nkv), _i(d), _i(K), _stream()), "gemm_qkv_rope")


def qkv_norm_rope_small_m_supported(M: int, K: int, d: int, rotary: int) -> bool:
    """Up to 8 rows (a row a warp; with 16, the norm that every block repeats costs more than
    the launch it saves: 1.03 against 0.92 ms a step), K a multiple of 32 up to 1024."""
    return 0 < M <= 8 and K % 32 == 0 and K <= 1024 and d % 16 == 0 and rotary == d


def qkv_norm_rope_small_m(x, x_out, delta, gain, eps, w, bias, pos, slot, cos, sin, q_out, k_pool,
                          v_pool, nh, nkv, d) -> None:
    """`qkv_rope_small_m` with the residual add and the RMS norm in front computed by the
    kernel itself: x_out = x + delta (delta as for rms_norm: [M, K], float32 partial sums
    [S, M, K], or None), projection of norm(x_out) * gain."""
    M, K = x.shape
    if x.dtype != torch.float32 or x_out.dtype != torch.float32 or x_out.shape != x.shape:
        raise ValueError("qkv_norm_rope_small_m: the residual stream is float32, in and out of one shape")
    if w.shape != ((nh + 2 * nkv) * d, K) or w.dtype != torch.bfloat16:
        raise ValueError("qkv_norm_rope_small_m: w is the stacked [(heads + 2 kv heads) d, K] weight")
    if not qkv_norm_rope_small_m_supported(M, K, d, 2 * cos.shape[1]):
        raise ValueError("qkv_norm_rope_small_m: sizes it does not take")
    n_partials, stride = _partials(delta, x)
    _check(_lib("linear_small_m").tokb200_qkv_norm_rope_small_m(
        _ptr(x), _ptr(x_out), _ptr(delta), _i(1 if delta is not None and delta.dtype == torch.float32 else 0),
        _i(n_partials), _ll(stride), _ptr(gain), _f(eps), _ptr(w), _ptr(bias), _ptr(pos), _ptr(slot),
        _ptr(cos), _ptr(sin), _ptr(q_out), _ptr(k_pool), _ptr(v_pool), _i(M), _i(nh), _i(nkv), _i(d),
        _i(K), _stream()), "qkv_norm_rope_small_m")


WIDE_TILE_ROWS = 128


def attention_tcgen05_supported(nh: int, nkv: int, d: int) -> bool:
    return d in (64, 128) and nh % nkv == 0


def attention_tcgen05(q, k_pool, v_pool, out, block_table, row_req, pos, tiles, n_tiles, nh, nkv, d,
                      page, window, scale) -> None:
    """Attention for portions of prompts on tcgen05 (bfloat16, head size 64 or 128).
    `tiles` is int32 [n, 2]: (first row, rows <= 128) of consecutive rows of one request."""
    if q.dtype != torch.bfloat16:
        raise ValueError("attention_tcgen05 is the bfloat16 kernel")
    if not attention_tcgen05_supported(nh, nkv, d):
        raise ValueError(f"attention_tcgen05: head size {d} is not taken (64 or 128)")
    lib = _load("attention_tcgen05.cu", defines=(f"HEAD_DIM={d}",))
    _check(lib.tokb200_attention_tcgen05(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(block_table),
        _i(block_table.shape[1]), _ptr(row_req), _ptr(pos), _ptr(tiles), _i(n_tiles), _i(nh),
        _i(nkv), _i(d), _i(page), _i(-1 if window is None else int(window)), _f(scale), _stream()),
        "attention_tcgen05")


def attention_tcgen05_check(d: int) -> None:
    flag = _load("attention_tcgen05.cu", defines=(f"HEAD_DIM={d}",)).tokb200_attention_tcgen05_error()
    if flag:
        raise KernelError("attention_tcgen05: a wait on the device ran out (status %d)" % flag)


# --------------------------------------------------------------------------- #
# a whole decoder layer of few rows in one kernel
class _LayerArgs(ctypes.Structure):
    _fields_ = (
        [(n, ctypes.c_void_p) for n in ("w_qkv", "b_qkv", "w_o", "gain1", "gain2", "w_gu", "w_d", "k_pool",
                                        "v_pool", "k_read", "v_read", "cos_t", "sin_t")] +
        [("eps1", ctypes.c_float), ("eps2", ctypes.c_float), ("scale", ctypes.c_float),
         ("window", ctypes.c_int), ("activation", ctypes.c_int),
         ("x_in", ctypes.c_void_p), ("delta", ctypes.c_void_p), ("delta_is_f32", ctypes.c_int),
         ("n_partials", ctypes.c_int), ("partial_stride", ctypes.c_longlong)] +
        [(n, ctypes.c_void_p) for n in ("x_mid", "x_out", "out", "pos", "slot", "row_req", "block_table")] +
        [("table_stride", ctypes.c_int), ("page", ctypes.c_int)] +
        [(n, ctypes.c_void_p) for n in ("q_buf", "att_part", "att_count", "att_out", "o_part", "act", "sync")] +
        [(n, ctypes.c_int) for n in ("M", "H", "I", "nh", "nkv", "d")] +
        [("stamps", ctypes.c_void_p), ("next_w_qkv", ctypes.c_void_p), ("next_gain1", ctypes.c_void_p),
         ("next_b_qkv", ctypes.c_void_p), ("repeat", ctypes.c_int)])


LAYER_HEAD_DIMS = (64, 128)
LAYER_MAX_ROWS = 32
LAYER_MAX_SPLITS = 32
_layer_plans = {}
# compile-time switches of the layer kernel's library (a test builds it with short wait limits)
_LAYER_DEFINES = ()


def _layer_lib(d: int):
    return _load("layer_small_m.cu", defines=(f"HEAD_DIM={d}",) + tuple(_LAYER_DEFINES))


def layer_small_m_splits(M: int, hidden: int, inner: int, nh: int, nkv: int, d: int):
    """(partial sums of the feed-forward, partial sums of the output projection) that the
    whole-layer kernel of few rows writes for these sizes on this device; (0, 0) when it does
    not take them (more than 32 rows, a head size it is not built for, hidden not a multiple
    of 32 or beyond 4096, inner not a multiple of 128, groups of more than 16 heads, too
    little shared memory for its ring)."""
    if M < 1 or M > LAYER_MAX_ROWS or d not in LAYER_HEAD_DIMS:
        return 0, 0
    key = (torch.cuda.current_device(), (M > 8) + (M > 16), hidden, inner, nh, nkv, d)
    if key not in _layer_plans:
        o_splits = ctypes.c_int(0)
        down = int(_layer_lib(d).tokb200_layer_small_m_splits(_i(M), _i(hidden), _i(inner), _i(nh), _i(nkv),
                                                              ctypes.byref(o_splits)))
        _layer_plans[key] = (down, int(o_splits.value))
    return _layer_plans[key]


def layer_small_m(x_in, delta, x_mid, x_out, out, gain1, eps1, w_qkv, b_qkv, pos, slot, row_req, block_table,
                  cos, sin, k_pool, v_pool, writes: bool, w_o, gain2, eps2, w_gate_up, w_down, nh: int,
                  nkv: int, d: int, page: int, window, scale: float, activation: str = "silu",
                  stamps: Optional[torch.Tensor] = None, next_layer=None, repeat: int = 1) -> None:
    """One pre-norm decoder layer for up to 32 rows of one token each (bfloat16): x_mid = x_in +
    delta; attention (q/k/v with bias, rotary encoding, cache write when `writes`, softmax over
    the paged keys) of rms_norm(x_mid) * gain1; x_out = x_mid + its output projection; out
    [S, M, H] = float32 partial sums over k of the gated feed-forward of rms_norm(x_out) * gain2.
    `delta` as for rms_norm ([M, H], float32 partial sums [S, M, H], or None); `w_gate_up` in the
    row order of `interleave_gate_up`; `out` has `layer_small_m_splits(...)[0]` planes.  `stamps`
    (int64 [blocks, 16], for profiling) receives the time in ns at which each block passes each phase;
    `next_layer` = (q/k/v weight of the same shape, first gain, q/k/v bias or None) of the layer that
    runs next: what that layer's kernel starts with is brought into L2 ahead."""
    M, hidden = x_in.shape
    inner = w_down.shape[1]
    down_splits, o_splits = layer_small_m_splits(M, hidden, inner, nh, nkv, d)
    if down_splits == 0:
        raise ValueError(f"layer_small_m does not take {M} rows of {hidden}, inner {inner}, {nh}/{nkv} heads of {d}")
    for t in (x_in, x_mid, x_out):
        if t.dtype != torch.float32 or tuple(t.shape) != (M, hidden):
            raise ValueError("layer_small_m: the residual stream is float32 [M, H], in, middle and out")
    if tuple(out.shape) != (down_splits, M, hidden) or out.dtype != torch.float32:
        raise ValueError(f"layer_small_m: out must be float32 {(down_splits, M, hidden)}")
    q_width = nh * d
    if w_qkv.dtype != torch.bfloat16 or tuple(w_qkv.shape) != ((nh + 2 * nkv) * d, hidden) or \
            tuple(w_o.shape) != (hidden, q_width) or tuple(w_gate_up.shape) != (2 * inner, hidden) or \
            tuple(w_down.shape) != (hidden, inner) or w_o.dtype != torch.bfloat16 or \
            w_gate_up.dtype != torch.bfloat16 or w_down.dtype != torch.bfloat16:
        raise ValueError("layer_small_m: bfloat16 weights [(nh + 2 nkv) d, H], [H, nh d], [2 I, H], [H, I]")
    if cos.shape[1] != d // 2 or k_pool.dtype != torch.bfloat16:
        raise ValueError("layer_small_m: the whole head is rotated, and the cache is bfloat16")
    n_partials, stride = _partials(delta, x_in)
    key = (x_in.device.index, M, hidden, inner, nh, nkv, d)
    if key not in _space.layer:
        dev = x_in.device
        _space.layer[key] = dict(
            q_buf=torch.empty((M, q_width), dtype=torch.bfloat16, device=dev),
            att_part=torch.empty((M, nh, LAYER_MAX_SPLITS, d + 2), dtype=torch.float32, device=dev),
            att_count=torch.zeros(M * nkv, dtype=torch.int32, device=dev),
            att_out=torch.zeros((M, q_width), dtype=torch.bfloat16, device=dev),
            o_part=torch.empty((o_splits, M, hidden), dtype=torch.float32, device=dev),
            act=torch.empty((LAYER_MAX_ROWS, inner), dtype=torch.bfloat16, device=dev),
            sync=torch.zeros(2, dtype=torch.int32, device=dev))
    sc = _space.layer[key]

    def ptr(t):
        return _ptr(t).value

    args = _LayerArgs(
        w_qkv=ptr(w_qkv), b_qkv=ptr(b_qkv), w_o=ptr(w_o), gain1=ptr(gain1), gain2=ptr(gain2),
        w_gu=ptr(w_gate_up), w_d=ptr(w_down), k_pool=ptr(k_pool) if writes else None,
        v_pool=ptr(v_pool) if writes else None, k_read=ptr(k_pool), v_read=ptr(v_pool), cos_t=ptr(cos),
        sin_t=ptr(sin), eps1=eps1, eps2=eps2, scale=scale, window=-1 if window is None else int(window),
        activation=activation_tag(activation), x_in=ptr(x_in), delta=ptr(delta),
        delta_is_f32=1 if delta is not None and delta.dtype == torch.float32 else 0, n_partials=n_partials,
        partial_stride=stride, x_mid=ptr(x_mid), x_out=ptr(x_out), out=ptr(out), pos=ptr(pos),
        slot=ptr(slot) if writes else None, row_req=ptr(row_req), block_table=ptr(block_table),
        table_stride=block_table.shape[1], page=page, q_buf=ptr(sc["q_buf"]), att_part=ptr(sc["att_part"]),
        att_count=ptr(sc["att_count"]), att_out=ptr(sc["att_out"]), o_part=ptr(sc["o_part"]),
        act=ptr(sc["act"]), sync=ptr(sc["sync"]), M=M, H=hidden, I=inner, nh=nh, nkv=nkv, d=d,
        stamps=ptr(stamps), repeat=repeat)
    if next_layer is not None and next_layer[0].shape == w_qkv.shape:
        args.next_w_qkv, args.next_gain1 = ptr(next_layer[0]), ptr(next_layer[1])
        args.next_b_qkv = ptr(next_layer[2])
    _check(_layer_lib(d).tokb200_layer_small_m(ctypes.byref(args), _stream()), "layer_small_m")


def layer_small_m_check(d: int) -> None:
    flag = _layer_lib(d).tokb200_layer_small_m_error()
    if flag:
        raise KernelError("layer_small_m: a wait on the device ran out (status %d)" % flag)


# ---- few rows, a large weight: one block a multiprocessor streams it through rings in shared memory ----
RING_ELEMENTS = 13_000_000     # from this many weight elements on (26 MB) the ring kernel leads the one with plain loads
RING_MAX_ROWS = 32
_RING = os.environ.get("TOKB200_RING", "1") != "0"     # TOKB200_RING=0: large weights on linear_small_m too
_ring_plans = {}


def linear_ring_supported(M: int, N: int, K: int, k_splits: int = 1, gated: bool = False) -> bool:
    """Sizes `linear_ring` / its gated form take on this device (up to 32 rows, K a multiple of 8 with at
    least 512 per piece of k, x's piece of k and the rings within a block's shared memory)."""
    if not (0 < M <= RING_MAX_ROWS and N > 0 and K > 0 and K % 8 == 0):
        return False
    key = (torch.cuda.current_device(), (M > 8) + (M > 16), N, K, k_splits, gated)
    if key not in _ring_plans:
        _ring_plans[key] = bool(_lib("linear_ring").tokb200_linear_ring_supported(
            _i(M), _i(N), _i(K), _i(k_splits), _i(1 if gated else 0)))
    return _ring_plans[key]


def linear_ring_splits(M: int, N: int, K: int, sms: int) -> int:
    """Pieces of k for a product whose consumer takes partial sums: the count (1 to 8) whose units of
    work (row tiles x pieces) divide most evenly over one block a multiprocessor, among those the
    kernel takes; 0 if it takes none."""
    tiles = -(-N // 16)
    best, best_waste = 0, None
    for s in range(1, 9):
        if not linear_ring_supported(M, N, K, s):
            continue
        units = tiles * s
        rounds = -(-units // sms)
        waste = rounds * sms / units
        if best_waste is None or waste < best_waste - 0.02:
            best, best_waste = s, waste
    return best


def linear_ring(x, w, bias, out, k_splits: int = 1) -> None:
    """out = x @ w.T (+ bias) for up to 16 rows and a large weight (bfloat16 in; out [M,N]
    bfloat16/float32, or float32 partial sums [k_splits, M, N] without bias)."""
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise ValueError("linear_ring: bfloat16 x [M,K] and w [N,K]")
    if not linear_ring_supported(M, N, K, k_splits):
        raise ValueError(f"linear_ring does not take {M} rows, {N} x {K}, {k_splits} pieces of k")
    if k_splits > 1:
        if tuple(out.shape) != (k_splits, M, N) or out.dtype != torch.float32 or bias is not None:
            raise ValueError("linear_ring: partial sums are float32 [S,M,N] without bias")
    elif tuple(out.shape) != (M, N) or out.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("linear_ring: out is [M,N] bfloat16 or float32")
    _check(_lib("linear_ring").tokb200_linear_ring(
        _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _i(1 if out.dtype == torch.float32 else 0), _i(M), _i(N), _i(K),
        _i(k_splits), _stream()), "linear_ring")


def linear_ring_gated(x, w, out, activation: str = "silu") -> None:
    """out[M, N/2] = act(x Wg^T) * (x Wu^T) for w from `interleave_gate_up`, up to 16 rows, a large weight."""
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or \
            w.shape[1] != K or tuple(out.shape) != (M, N // 2):
        raise ValueError("linear_ring_gated: bfloat16 x [M,K], w [N,K], out [M,N/2]")
    if not linear_ring_supported(M, N, K, 1, True):
        raise ValueError(f"linear_ring_gated does not take {M} rows, {N} x {K}")
    _check(_lib("linear_ring").tokb200_linear_ring_gated(
        _ptr(x), _ptr(w), _ptr(out), _i(M), _i(N), _i(K), _i(activation_tag(activation)), _stream()),
        "linear_ring_gated")


# ---- read-only streams in the decoding kernels' access patterns (bench.py --stream-probe) ----
STREAM_PATTERNS = {"coalesced": 0, "fragment": 1, "fragment_wide": 2}


def stream_probe_loads(w: torch.Tensor, pattern: str, in_flight: int, blocks: int, sink: torch.Tensor) -> None:
    """Read the bfloat16 matrix `w` [N, K] once with plain loads in one of STREAM_PATTERNS,
    `in_flight` (2, 4 or 8) steps of loads a thread, from `blocks` blocks of 256 threads."""
    N, K = w.shape
    _check(_lib("stream_probe").tokb200_stream_probe_loads(
        _ptr(w), _i(N), _i(K), _i(STREAM_PATTERNS[pattern]), _i(in_flight), _i(blocks), _ptr(sink), _stream()),
        "stream_probe_loads")


def stream_probe_bulk(w: torch.Tensor, piece_bytes: int, rows_per_stage: int, stages: int, blocks: int,
                      sink: torch.Tensor) -> None:
    """Read `w` once through a ring of shared-memory stages filled by bulk copies of `piece_bytes`
    of a row each (a stage: `rows_per_stage` pieces), one producer and one consumer warp a block."""
    N, K = w.shape
    _check(_lib("stream_probe").tokb200_stream_probe_bulk(
        _ptr(w), _i(N), _i(K), _i(piece_bytes), _i(rows_per_stage), _i(stages), _i(blocks), _ptr(sink), _stream()),
        "stream_probe_bulk")


def stream_probe_async_ring(w: torch.Tensor, depth: int, blocks: int, sink: torch.Tensor) -> None:
    """Read `w` once in the fragment pattern through rings of `depth` (4, 6 or 8) shared-memory
    stages a warp, filled by 16-byte asynchronous copies."""
    N, K = w.shape
    _check(_lib("stream_probe").tokb200_stream_probe_async_ring(
        _ptr(w), _i(N), _i(K), _i(depth), _i(blocks), _ptr(sink), _stream()), "stream_probe_async_ring")
