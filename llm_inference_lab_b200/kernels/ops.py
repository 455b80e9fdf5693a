"""Python face of the CUDA kernels.

Each function checks shapes and types on the host, then calls one ``extern "C"``
entry point of a library built from ``csrc/kernels`` on the current CUDA stream.
There is no fallback: without a GPU, or without the built library, a call
raises.  Tensors are torch tensors on the GPU; a kernel never allocates.
"""
from __future__ import annotations

import ctypes
import threading

import torch

from . import build

F32, BF16 = 0, 1
_libs: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelError(RuntimeError):
    pass


DEVICE_ERRORS = {1: "a page or slot index outside the pool", 2: "a bounded wait inside a kernel ran out",
                 3: "a gathered row index outside the batch"}


_fast: dict = {}    # (name, values of the defines) -> library handle; read without the lock on the hot path


def lib(name: str, defines: dict[str, int] | None = None) -> ctypes.CDLL:
    fast_key = (name, tuple(defines.values()) if defines else None)
    handle = _fast.get(fast_key)
    if handle is not None:
        return handle
    key = name + repr(sorted((defines or {}).items()))
    with _lock:
        if key in _libs:
            _fast[fast_key] = _libs[key]
            return _libs[key]
    path = build.kernel_library(name, defines)
    handle = ctypes.CDLL(path)
    with _lock:
        _libs[key] = handle
        _fast[fast_key] = handle
    return handle


def require_gpu() -> None:
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: the engine runs on a B200 only and has no CPU fallback")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported storage type {dtype}: the kernels take float32 or bfloat16")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> ctypes.c_void_p:
    """The current CUDA stream's handle (also the capturing stream while a graph is recorded)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def copy_to_device(dst: torch.Tensor, pinned_src: torch.Tensor, words_from: int, words_to: int) -> None:
    """dst[words_from:words_to] = pinned_src[words_from:words_to] (both int32, same layout) on the current
    stream, without the host-side cost of a tensor copy."""
    _check(lib("rowwise").lab_copy_to_device(
        ctypes.c_void_p(dst.data_ptr() + 4 * words_from), ctypes.c_void_p(pinned_src.data_ptr() + 4 * words_from),
        ctypes.c_longlong(4 * (words_to - words_from)), _stream()), "copy_to_device", 0)


_stream_objects: dict = {}


def current_stream() -> "torch.cuda.Stream":
    """torch's object for the current stream, found through its raw handle (the library's own
    lookup costs several microseconds a call)."""
    if _raw_stream is None:
        return torch.cuda.current_stream()
    device = torch.cuda.current_device()
    key = (device, _raw_stream(device))
    obj = _stream_objects.get(key)
    if obj is None:
        obj = _stream_objects[key] = torch.cuda.current_stream()
    return obj


def _ptr(t) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


class _Counter:
    """Kernel launches issued through this module (a graph replay adds what it captured)."""
    launches = 0


COUNTER = _Counter()


def _check(code: int, what: str, launches: int = 1) -> None:
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code}")
    COUNTER.launches += launches


def _on_gpu(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must be CUDA tensors")


_error_hooks: list = []


def on_device_error(method) -> None:
    """The bound method `method` is called when `take_device_errors` finds an error (to put scratch
    state right again); held weakly, so that it does not keep its object alive."""
    import weakref
    _error_hooks[:] = [h for h in _error_hooks if h() is not None]
    _error_hooks.append(weakref.WeakMethod(method))


def take_device_errors() -> None:
    """Synchronise and raise if any kernel left an error code."""
    for key, handle in list(_libs.items()):
        out = ctypes.c_int(0)
        _check(handle.lab_take_error_word(ctypes.byref(out)), "reading the error word", 0)
        if out.value:
            for hook in _error_hooks:
                method = hook()
                if method is not None:
                    method()
            raise KernelError(f"kernel library {key.split('[')[0]} reported: "
                              f"{DEVICE_ERRORS.get(out.value, out.value)}")


def wait_probe(limit_ms: float = 2.0) -> bool:
    """Runs the tensor-core product library's test kernel whose wait nothing ends, with a limit of
    `limit_ms` (50 at most).  Returns True if the wait gave up, as it must; the library's error word
    then says that a bounded wait ran out (`take_device_errors` raises)."""
    flag = torch.zeros((1,), dtype=torch.int32, device="cuda")
    _check(lib("gemm_tc").lab_gemm_tc_wait_probe(ctypes.c_ulonglong(int(limit_ms * 1e6)), _ptr(flag), _stream()),
           "wait_probe")
    return bool(flag.item())


# ----------------------------------------------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    _on_gpu(ids, table)
    tokens, (vocab, hidden) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((tokens, hidden), dtype=table.dtype, device=table.device)
    assert ids.dtype == torch.int32 and table.is_contiguous() and out.is_contiguous()
    _check(lib("rowwise").lab_embed(_ptr(out), _ptr(table), _ptr(ids), tokens, hidden, vocab,
                                    dtype_code(table.dtype), _stream()), "embed")
    return out


def add_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, delta: torch.Tensor | None = None,
                partial: torch.Tensor | None = None, rows: torch.Tensor | None = None,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """x += delta (+ sum of `partial` over its first axis), in place; returns rmsnorm(x) * weight.

    With `rows`, output row i is computed from x[rows[i]] and x is left as it is.
    """
    _on_gpu(x, weight, delta, partial, rows)
    n_in, hidden = x.shape
    n_out = n_in if rows is None else rows.numel()
    if out is None:
        out = torch.empty((n_out, hidden), dtype=x.dtype, device=x.device)
    assert x.is_contiguous() and weight.dtype == x.dtype and weight.numel() == hidden
    assert delta is None or (delta.shape == x.shape and delta.dtype == x.dtype and delta.is_contiguous())
    splits, stride = 0, 0
    if partial is not None:
        assert partial.dtype == torch.float32 and partial.is_contiguous() and partial.shape[1:] == x.shape
        splits, stride = partial.shape[0], n_in * hidden
    _check(lib("rowwise").lab_add_rmsnorm(_ptr(out), _ptr(x), _ptr(delta), _ptr(partial), splits,
                                          ctypes.c_longlong(stride), _ptr(weight), _ptr(rows), n_out, n_in, hidden,
                                          ctypes.c_float(eps), dtype_code(x.dtype), _stream()), "add_rmsnorm")
    return out


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor | None, inv_freq: torch.Tensor, rotary_dim: int,
                  slots: torch.Tensor | None, cache_k: torch.Tensor | None, cache_v: torch.Tensor | None,
                  n_q: int, n_kv: int, head_dim: int, bias: torch.Tensor | None = None,
                  q_out: torch.Tensor | None = None) -> torch.Tensor:
    """Rotate q and k, and write k and v to their cache slots.  Returns the rotated q.

    `qkv` is the fused projection [tokens, (n_q + 2 n_kv) * d] rounded to the storage type (q is
    rotated in place and the q columns are returned), or its 32-bit split-K partial products
    [splits, tokens, ...] with `bias` still to add (rotated q goes to a new tensor).
    """
    _on_gpu(qkv, positions, inv_freq, slots, cache_k, cache_v, bias, q_out)
    width = (n_q + 2 * n_kv) * head_dim
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2
    assert positions is not None or rotary_dim == 0
    page_size = num_pages = 0
    if cache_k is not None:
        num_pages, kvh, page_size, d = cache_k.shape
        assert kvh == n_kv and d == head_dim and cache_k.is_contiguous() and cache_v.is_contiguous()
        assert cache_v.shape == cache_k.shape and slots is not None
    if qkv.dim() == 3:
        splits, tokens = qkv.shape[0], qkv.shape[1]
        assert qkv.dtype == torch.float32 and qkv.is_contiguous() and qkv.shape[2] == width
        dt = cache_k.dtype if cache_k is not None else torch.bfloat16
        if q_out is None:
            q_out = torch.empty((tokens, n_q * head_dim), dtype=dt, device=qkv.device)
        _check(lib("rowwise").lab_rope_kv_write(
            None, width, _ptr(qkv), splits, ctypes.c_longlong(tokens * width), _ptr(bias), _ptr(q_out),
            _ptr(positions), _ptr(inv_freq), rotary_dim, _ptr(slots), _ptr(cache_k), _ptr(cache_v), tokens, n_q, n_kv,
            head_dim, page_size, num_pages, dtype_code(dt), _stream()), "rope_kv_write")
        return q_out
    tokens = qkv.shape[0]
    assert qkv.stride(1) == 1 and qkv.shape[1] == width and bias is None
    assert cache_k is None or cache_k.dtype == qkv.dtype
    _check(lib("rowwise").lab_rope_kv_write(
        _ptr(qkv), qkv.stride(0), None, 0, ctypes.c_longlong(0), None, None, _ptr(positions), _ptr(inv_freq),
        rotary_dim, _ptr(slots), _ptr(cache_k), _ptr(cache_v), tokens, n_q, n_kv, head_dim, page_size, num_pages,
        dtype_code(qkv.dtype), _stream()), "rope_kv_write")
    return qkv[:, : n_q * head_dim]


_no_freq: dict = {}


def kv_store(qkv: torch.Tensor, slots, cache_k, cache_v, n_q: int, n_kv: int, head_dim: int) -> torch.Tensor:
    """The framework's paged store: writes the k and v columns of the fused projection `qkv`
    [tokens, (n_q + 2 n_kv) * d] to their cache slots (nothing if `cache_k` is None) and returns the q
    columns.  What a position encoding that only encodes leaves to the framework."""
    key = str(qkv.device)
    none = _no_freq.get(key)
    if none is None:
        none = _no_freq[key] = torch.zeros((0,), dtype=torch.float32, device=qkv.device)
    return rope_kv_write(qkv, None, none, 0, slots, cache_k, cache_v, n_q, n_kv, head_dim)


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """(cos, sin) of pos * inv_freq for every row of a step: [tokens, rotary_dim / 2, 2] float32."""
    tokens, half = positions.numel(), inv_freq.numel()
    table = torch.empty((tokens, half, 2), dtype=torch.float32, device=positions.device)
    _check(lib("rowwise").lab_rope_table(_ptr(table), _ptr(positions), _ptr(inv_freq), tokens, half, _stream()),
           "rope_table")
    return table


def rope_kv_write_table(qkv, table, rotary_dim, slots, cache_k, cache_v, n_q, n_kv, head_dim) -> torch.Tensor:
    """The rotation and cache write for bfloat16 steps with many rows, with cos/sin from `rope_table`."""
    tokens = qkv.shape[0]
    page_size = num_pages = 0
    if cache_k is not None:
        num_pages, _, page_size, _ = cache_k.shape
    _check(lib("rowwise").lab_rope_kv_write_table(
        _ptr(qkv), qkv.stride(0), _ptr(table), rotary_dim, _ptr(slots), _ptr(cache_k), _ptr(cache_v), tokens, n_q,
        n_kv, head_dim, page_size, num_pages, _stream()), "rope_kv_write_table")
    return qkv[:, : n_q * head_dim]


def gemm_plain(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, gated: bool = False,
               out_f32: bool = False, out: torch.Tensor | None = None, gelu: bool = False,
               gate_limit: float = 0.0) -> torch.Tensor:
    """out = x @ w.T (+ bias) on the ordinary arithmetic units; `gated`: silu(x@wg.T) * (x@wu.T), w = [wg; wu]
    (`gate_limit` > 0: the capped form, see `linear_gated`); `gelu`: the tanh form of GELU after the bias, before
    the rounding."""
    assert not (gated and gelu)
    _on_gpu(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0] // 2 if gated else w.shape[0]
    assert w.shape[1] == K and w.is_contiguous() and x.stride(1) == 1 and w.dtype == x.dtype
    assert bias is None or (bias.dtype == x.dtype and bias.numel() == N and not gated)
    odt = torch.float32 if (out_f32 or x.dtype == torch.float32) else x.dtype
    if out is None:
        out = torch.empty((M, N), dtype=odt, device=x.device)
    assert out.dtype == odt and out.stride(1) == 1 and out.shape == (M, N)
    _check(lib("gemm_plain").lab_gemm_plain(_ptr(out), _ptr(x), _ptr(w), _ptr(bias), M, N, K, x.stride(0),
                                            out.stride(0), (1 + int(gelu)) if gelu else int(gated), dtype_code(x.dtype), int(out_f32),
                                            ctypes.c_float(gate_limit), _stream()),
           "gemm_plain")
    return out


def linear_heads(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, h, :] = w[h] @ x[t, h, :] for every head h: x [tokens, heads, >= k] (a head's first k entries are
    read), w [heads, n, k] contiguous, out [tokens, heads, >= n] (a head's first n entries are written), 32-bit
    or of x's type.  Steps of many bfloat16 tokens run one tensor-core product per head; else all heads are
    one launch on the ordinary units."""
    _on_gpu(x, w, out)
    tokens, heads = x.shape[0], x.shape[1]
    n, k = w.shape[1], w.shape[2]
    assert w.is_contiguous() and w.shape[0] == heads and w.dtype == x.dtype and x.stride(2) == 1 and out.stride(2) == 1
    assert x.stride(0) == heads * x.stride(1) and out.stride(0) == heads * out.stride(1)
    assert out.dtype in (x.dtype, torch.float32) and x.shape[2] >= k and out.shape[2] >= n
    f32 = out.dtype == torch.float32
    if x.dtype == torch.bfloat16 and tokens > 128 and not _force_plain:
        for h in range(heads):
            linear(x[:, h, :k], w[h], None, out_f32=f32, out=out[:, h, :n])
        return out
    _check(lib("gemm_plain").lab_gemm_plain_batched(
        _ptr(out), _ptr(x), _ptr(w), tokens, n, k, x.stride(0), out.stride(0), heads, ctypes.c_longlong(x.stride(1)),
        ctypes.c_longlong(n * k), ctypes.c_longlong(out.stride(1)), dtype_code(x.dtype), int(f32), _stream()),
        "gemm_plain_batched")
    return out


def attention_plain(q: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, row_req: torch.Tensor,
                    row_pos: torch.Tensor, block_table: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                    window: int, scale: float, out: torch.Tensor | None = None, keep_first: int = 0,
                    sink_one: bool = False, sink: torch.Tensor | None = None,
                    dist_bias: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of every row over its request's pages; q may be a column slice of the fused projection.
    `keep_first`: with a window, the first that many positions stay visible; `sink_one`: one more in the
    softmax's denominator; `sink` [n_q] 32-bit: exp(sink[h]) more instead; `dist_bias` [n_q, L] 32-bit: added to
    the scaled score by distance query - key, distances from L - 1 on sharing the last entry."""
    _on_gpu(q, cache_k, cache_v, row_req, row_pos, block_table, sink, dist_bias)
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() >= n_q and sink.is_contiguous())
    assert dist_bias is None or (dist_bias.dtype == torch.float32 and dist_bias.dim() == 2 and
                                 dist_bias.shape[0] == n_q and dist_bias.is_contiguous())
    tokens = q.shape[0]
    if out is None:
        out = torch.empty((tokens, n_q * head_dim), dtype=q.dtype, device=q.device)
    num_pages, kvh, page_size, d = cache_k.shape
    assert kvh == n_kv and d == head_dim and q.stride(1) == 1 and cache_k.dtype == q.dtype
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous()
    _check(lib("attention_plain").lab_attention_plain(
        _ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(cache_k), _ptr(cache_v), _ptr(row_req), _ptr(row_pos),
        _ptr(block_table), block_table.shape[1], tokens, n_q, n_kv, head_dim, page_size, num_pages, window,
        ctypes.c_float(scale), int(keep_first), int(bool(sink_one) or sink is not None), _ptr(sink), _ptr(dist_bias),
        dist_bias.shape[1] if dist_bias is not None else 0, dtype_code(q.dtype), _stream()), "attention_plain")
    return out


_sample_scratch: dict = {}
# Scratch that was outgrown stays alive: a CUDA graph captured earlier still launches kernels with its address.
_retired_scratch: list = []


def _sample_buffers(device, rows: int, chunks: int):
    """Scratch of the sampling kernel, kept per device (its counters must stay zero between calls)."""
    key = str(device)
    need = rows * chunks
    buf = _sample_scratch.get(key)
    if buf is None or buf[0].numel() < need or buf[2].numel() < rows:
        cap_rows, cap = max(rows, 256), max(need, 256 * chunks)
        buf = (torch.empty((cap,), dtype=torch.float32, device=device),
               torch.empty((cap,), dtype=torch.int32, device=device),
               torch.zeros((cap_rows,), dtype=torch.int32, device=device))
        _retired_scratch.append(_sample_scratch.get(key))
        _sample_scratch[key] = buf
    return buf


def sample(logits: torch.Tensor, temperature: torch.Tensor | None = None, seeds: torch.Tensor | None = None,
           positions: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of 32-bit logits: greedy where temperature is 0 (or None), else Gumbel-max."""
    _on_gpu(logits, temperature, seeds, positions)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    if temperature is not None:
        assert temperature.dtype == torch.float32 and seeds.dtype == torch.int32 and positions.dtype == torch.int32
        assert temperature.numel() == rows and seeds.numel() == rows and positions.numel() == rows
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    L = lib("sampling")
    chunks = L.lab_sample_chunks(vocab)
    pv = pi = cnt = None
    if chunks > 1:
        pv, pi, cnt = _sample_buffers(logits.device, rows, chunks)
    _check(L.lab_sample(_ptr(out), _ptr(logits), ctypes.c_longlong(logits.stride(0)), rows, vocab, _ptr(temperature),
                        _ptr(seeds), _ptr(positions), _ptr(pv), _ptr(pi), _ptr(cnt), _stream()), "sample")
    return out


# ----------------------------------------------------------------------------------------
# Dispatch: which kernel serves a matrix product or an attention call.
#
# float32 always runs the plain kernels (a true 32-bit path: no tensor cores, no reduced
# precision).  bfloat16 runs the tensor-core kernels; `force_plain(True)` sends bfloat16 to
# the plain kernels as well, which tests use to tell a kernel fault from a model fault.
# ----------------------------------------------------------------------------------------
_force_plain = False
_sm_count = 0


def sm_count() -> int:
    """Streaming multiprocessors of the current device (the host's choices of tiles and splits go by
    it, as the kernels' own grids do); 148, a B200's, where no device is present."""
    global _sm_count
    if _sm_count == 0:
        if torch.cuda.is_available():
            _sm_count = int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
        else:
            _sm_count = 148
    return _sm_count


def forced_plain() -> bool:
    return _force_plain


def force_plain(flag: bool) -> bool:
    global _force_plain
    old, _force_plain = _force_plain, bool(flag)
    return old


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, gated: bool = False,
            out_f32: bool = False, swap: bool | None = None, bn: int | None = None, splits: int = 1,
            out: torch.Tensor | None = None, gelu: bool = False, gate_limit: float = 0.0) -> torch.Tensor:
    """out = x @ w.T (+ bias) on the tcgen05 tensor cores (bfloat16 in, 32-bit accumulate); `gelu`: the
    tanh form of GELU after the bias, before the rounding (not with `gated` or `splits`).

    `swap` puts output features on the M side of the MMA (few tokens); `bn` is the tile on the
    other side; `splits` > 1 returns 32-bit partial products [splits, tokens, out].
    """
    _on_gpu(x, w, bias, out)
    T, K = x.shape
    n_out = w.shape[0] // 2 if gated else w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc takes bfloat16 operands")
    if K % 8 or x.stride(0) % 8 or x.stride(1) != 1 or not w.is_contiguous() or w.shape[1] != K:
        raise KernelError(f"gemm_tc: K={K} and the row stride must be multiples of 8 (16-byte rows for TMA)")
    if x.data_ptr() % 16 or w.data_ptr() % 16:
        raise KernelError("gemm_tc: operands must start on a 16-byte boundary")
    if swap is None:
        swap = T <= (64 if gated else 128)
    if bn is None:
        if swap:
            bn = 16
            while bn < min(T, 64 if gated else 256):
                bn *= 2
        else:
            bn = 256 if gated else 128
    if splits > 1:
        if gated or bias is not None:
            raise KernelError("split-K takes no bias and no gate")
        k_tiles = -(-K // 64)
        per = -(-k_tiles // splits)
        splits = -(-k_tiles // per)       # no empty split
    if splits > 1:
        out = torch.empty((splits, T, n_out), dtype=torch.float32, device=x.device) if out is None else out
        ld_out, f32 = n_out, True
    else:
        odt = torch.float32 if out_f32 else torch.bfloat16
        if out is None:
            out = torch.empty((T, n_out), dtype=odt, device=x.device)
        assert out.dtype == odt and out.stride(1) == 1
        ld_out, f32 = out.stride(0), out_f32
    if gelu and (gated or splits > 1):
        raise KernelError("gemm_tc: GELU goes with the plain, unsplit product")
    _check(lib("gemm_tc").lab_gemm_tc(_ptr(out), _ptr(x), _ptr(w), _ptr(bias), T, n_out, K, x.stride(0), ld_out,
                                      (1 + int(gelu)) if gelu else int(gated), int(f32), int(swap), bn, splits,
                                      ctypes.c_float(gate_limit), _stream()), "gemm_tc")
    return out


def gemm_tc2(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, gated: bool = False,
             out_f32: bool = False, splits: int = 1, out: torch.Tensor | None = None, bn: int = 0,
             gelu: bool = False, gate_limit: float = 0.0) -> torch.Tensor:
    """out = x @ w.T (+ bias) on pairs of SMs (tcgen05.mma.cta_group::2): tiles of 256 tokens by 256
    accumulator columns, each CTA of a pair loading half of the weight tile.  For steps with many
    tokens; `splits` > 1 returns 32-bit partial products [splits, tokens, out].  `bn`: accumulator
    columns of a tile (256, 224 or 192; 0: the width whose tiles fill the rounds of the pairs best)."""
    _on_gpu(x, w, bias, out)
    T, K = x.shape
    n_out = w.shape[0] // 2 if gated else w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc2 takes bfloat16 operands")
    if not _tc_operands(x, w) or w.shape[1] != K:
        raise KernelError(f"gemm_tc2: K={K} and the row stride must be multiples of 8 (16-byte rows for TMA)")
    if splits > 1:
        if gated or bias is not None:
            raise KernelError("split-K takes no bias and no gate")
        k_tiles = -(-K // 64)
        per = -(-k_tiles // splits)
        splits = -(-k_tiles // per)       # no empty split
    if splits > 1:
        out = torch.empty((splits, T, n_out), dtype=torch.float32, device=x.device) if out is None else out
        ld_out, f32 = n_out, True
    else:
        odt = torch.float32 if out_f32 else torch.bfloat16
        if out is None:
            out = torch.empty((T, n_out), dtype=odt, device=x.device)
        assert out.dtype == odt and out.stride(1) == 1
        ld_out, f32 = out.stride(0), out_f32
    if gelu and (gated or splits > 1):
        raise KernelError("gemm_tc2: GELU goes with the plain, unsplit product")
    _check(lib("gemm_tc2").lab_gemm_tc2(_ptr(out), _ptr(x), _ptr(w), _ptr(bias), T, n_out, K, x.stride(0), ld_out,
                                        (1 + int(gelu)) if gelu else int(gated), int(f32), splits, bn,
                                        ctypes.c_float(gate_limit), _stream()), "gemm_tc2")
    return out


def qkv_fusable(x, w, head_dim: int, rotary_dim: int) -> bool:
    """Whether `qkv_rope_store` serves this projection: bfloat16 operands the tensor-core product
    takes, heads of 64 or 128 (a head must lie whole inside a tile), rotation over the whole head."""
    return (x.dtype == torch.bfloat16 and not _force_plain and head_dim in (64, 128) and rotary_dim == head_dim
            and _tc_operands(x, w))


def qkv_rope_store(x, w_qkv, bias, table, slots, cache_k, cache_v, n_q: int, n_kv: int, head_dim: int,
                   bn: int | None = None) -> torch.Tensor:
    """The fused q/k/v projection with its epilogue in one kernel: x @ w_qkv.T + bias, rounded; q and k
    rotated with the cosines and sines of `table` ([tokens, head_dim / 2, 2] from `rope_table`); the
    rotated q returned [tokens, n_q * head_dim]; k and v written to their cache slots (`cache_k` None:
    the call does not write the cache).  Tokens lie on the 128-row side of the product: for steps of
    many tokens."""
    _on_gpu(x, w_qkv, bias, table, slots, cache_k, cache_v)
    T, K = x.shape
    width = (n_q + 2 * n_kv) * head_dim
    if not qkv_fusable(x, w_qkv, head_dim, head_dim):
        raise KernelError("qkv_rope_store takes bfloat16 operands with 16-byte rows and heads of 64 or 128")
    assert w_qkv.shape == (width, K) and (bias is None or (bias.numel() == width and bias.dtype == x.dtype))
    assert table.dtype == torch.float32 and table.is_contiguous() and table.shape == (T, head_dim // 2, 2)
    page_size = num_pages = 0
    if cache_k is not None:
        num_pages, kvh, page_size, d = cache_k.shape
        assert kvh == n_kv and d == head_dim and cache_k.is_contiguous() and cache_v.is_contiguous()
        assert cache_v.shape == cache_k.shape and cache_k.dtype == x.dtype and slots is not None
        assert slots.dtype == torch.int32 and slots.numel() >= T
    if bn is None:
        bn = _pick_prefill_tiles(T, width, K, False)[1]     # 128, or 256 where its waves cost less
    q = torch.empty((T, n_q * head_dim), dtype=x.dtype, device=x.device)
    _check(lib("gemm_tc").lab_gemm_tc_qkv(
        _ptr(q), _ptr(x), _ptr(w_qkv), _ptr(bias), T, n_q, n_kv, head_dim, K, x.stride(0), q.stride(0), _ptr(table),
        _ptr(slots), _ptr(cache_k), _ptr(cache_v), page_size, num_pages, bn, _stream()), "gemm_tc_qkv")
    return q


_pick_scratch: dict = {}
# Rows up to which a step's head picks its tokens itself (the kernel takes up to 128).  Measured at the
# Qwen2.5-0.5B sizes against the head that writes 32-bit logits for the sampling kernel: a decode step of
# 8 or 16 rows takes the same time (0.792 ms both ways; 0.812 against 0.814 ms) without the 5 to 10 MB of
# logits written and read back; at 32 rows the pick in the epilogue costs more than the logits' traffic
# (0.980 against 0.950 ms), at 64 rows 1.16 against 1.14 ms.
PICK_MAX_ROWS = 16


def head_pick_fusable(x, w) -> bool:
    """Whether `head_pick` serves this head: bfloat16 operands the tensor-core product takes, few rows."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and not _force_plain
            and x.shape[0] <= min(PICK_MAX_ROWS, 128) and _tc_operands(x, w))


def head_pick(x, w, temperature=None, seeds=None, positions=None, out=None) -> torch.Tensor:
    """One token per row of x from the head's logits x @ w.T without writing them: every tile of the
    product keeps its best candidate per row (greedy, or Gumbel-max where `temperature` > 0, by the
    sampling kernel's rule) and a second, tiny kernel picks each row's best."""
    _on_gpu(x, w, temperature, seeds, positions, out)
    T, K = x.shape
    vocab = w.shape[0]
    if not (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and T <= 128 and _tc_operands(x, w)):
        raise KernelError("head_pick takes bfloat16 operands with 16-byte rows and up to 128 rows")
    if temperature is not None:
        assert temperature.dtype == torch.float32 and seeds.dtype == torch.int32 and positions.dtype == torch.int32
        assert temperature.numel() >= T and seeds.numel() >= T and positions.numel() >= T
    if out is None:
        out = torch.empty((T,), dtype=torch.int32, device=x.device)
    assert out.dtype == torch.int32 and out.numel() >= T
    tiles = -(-vocab // 128)
    key = str(x.device)
    buf = _pick_scratch.get(key)
    if buf is None or buf[0].numel() < T * tiles:
        cap = max(T, 128) * tiles
        buf = (torch.empty((cap,), dtype=torch.float32, device=x.device),
               torch.empty((cap,), dtype=torch.int32, device=x.device))
        _retired_scratch.append(_pick_scratch.get(key))
        _pick_scratch[key] = buf
    bn = 16
    while bn < T:
        bn *= 2
    _check(lib("gemm_tc").lab_gemm_tc_pick(_ptr(out), _ptr(x), _ptr(w), T, vocab, K, x.stride(0), _ptr(temperature),
                                           _ptr(seeds), _ptr(positions), _ptr(buf[0]), _ptr(buf[1]), bn, _stream()),
           "gemm_tc_pick", 2)
    return out


def _pick_splits(T: int, n_out: int, K: int) -> int:
    """Split K when an output has too few tiles to keep the memory system busy (decode)."""
    if T > 128:
        return 1
    tiles = -(-n_out // 128)
    k_tiles = -(-K // 64)
    if tiles >= sm_count() // 2 or k_tiles < 8:
        return 1
    return max(1, min(-(-k_tiles // 4), sm_count() // tiles, 16))   # about 4 k-tiles per CTA (measured best)


def _pick_prefill_tiles(T: int, n_out: int, K: int, allow_partial: bool) -> tuple[str, int, int]:
    """(kernel, N tile, K splits) of a product with many tokens (tokens on the 128-row side);
    kernel is "pair" (two CTAs per 256 x 256 tile) or "tc".  Measured on the down and output
    projections of the 0.5B, 1.5B and 7B layer sizes at 256 to 4,096 tokens, together with the
    norm that sums the partial products:
    * a CTA fills shared memory from L2 at a limited rate, so tiles with more arithmetic per byte
      run closer to the tensor cores' pace: 128 x 128 tiles take about 420 cycles per 64 elements
      of K, 128 x 256 tiles 600, and a pair's 256 x 256 tile 900;
    * pairs win once there are enough tiles for most of the 74 pairs of SMs and K is long
      (down at 2,048 tokens, 1.5B: 61 against 75 us; 7B: 221 against 249 us);
    * while 128-wide tiles fill at most one wave, they win, with K split so that the wave is
      full and a split keeps 16 k-tiles or more (down at 2,048 tokens, 0.5B: 28 against 34 us
      for 256-wide tiles and two splits; at 512 tokens 15 against 21 us);
    * beyond one wave, the width whose waves cost less."""
    m_tiles, k_tiles = -(-T // 128), -(-K // 64)
    pairs = -(-T // 256) * (-(-n_out // 256))
    if k_tiles >= 32 and pairs >= 48:
        return "pair", 256, 1
    t128, t256 = m_tiles * (-(-n_out // 128)), m_tiles * (-(-n_out // 256))
    if t128 <= sm_count():
        splits = max(1, min(sm_count() // t128, k_tiles // 16)) if allow_partial else 1
        return "tc", 128, splits
    if -(-t256 // sm_count()) * 600 < -(-t128 // sm_count()) * 420:
        return "tc", 256, 1
    return "tc", 128, 1


def _tc_operands(x, w) -> bool:
    """Whether TMA can describe the operands: rows of 16-byte multiples that start on 16-byte
    boundaries.  Widths that are no multiple of 8 go to the plain kernel instead."""
    return (x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1 and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


# activations a plain product applies in its epilogue, with their codes (`gelu` = 1, 2 in the product kernels' faces)
ACTIVATIONS = {"gelu_tanh": 1, "relu2": 2}


def linear(x, w, bias=None, out_f32=False, allow_partial=False, out=None, act=None):
    """x @ w.T (+ bias).  With `allow_partial` the result may come back as 32-bit partial
    products [splits, tokens, out], without the bias, that the consumer sums (`add_rmsnorm`,
    `rope_kv_write`, `stream_add`).  `out`: where the result goes (rows may be strided).  `act`:
    an activation of the result ("gelu_tanh", or "relu2": the square of relu), applied after the bias and before the rounding."""
    if act is not None and (act not in ACTIVATIONS or allow_partial):
        raise KernelError(f"linear: activation {act!r} is not built, or asked of partial products")
    gelu = ACTIVATIONS[act] if act is not None else 0      # the epilogue's code of the activation
    if x.dtype == torch.float32 or _force_plain or not _tc_operands(x, w) or (
            out is not None and (out.stride(0) % 8 or out.data_ptr() % 16)):
        return gemm_plain(x, w, bias, out_f32=out_f32, out=out, gelu=gelu)
    T = x.shape[0]
    if T > 128:
        kind, bn, splits = _pick_prefill_tiles(T, w.shape[0], x.shape[1],
                                               allow_partial and bias is None and out is None)
        if kind == "pair":
            return gemm_tc2(x, w, bias, out_f32=out_f32, out=out, gelu=gelu)
        if splits > 1:
            return gemm_tc(x, w, None, swap=False, bn=bn, splits=splits)
        return gemm_tc(x, w, bias, out_f32=out_f32, swap=False, bn=bn, out=out, gelu=gelu)
    splits = _pick_splits(T, w.shape[0], x.shape[1]) if allow_partial and out is None else 1
    if splits > 1:
        return gemm_tc(x, w, None, splits=splits)     # the consumer adds the bias
    return gemm_tc(x, w, bias, out_f32=out_f32, out=out, gelu=gelu)


def linear_gated(x, w_gate_up, limit: float = 0.0):
    """silu(g) * u with g = x @ wg.T, u = x @ wu.T and w_gate_up = [wg; wu].  `limit` > 0: the capped form,
    g' = min(g, limit), u' = clamp(u, -limit, limit), g' * sigmoid(1.702 g') * (u' + 1)."""
    if x.dtype == torch.float32 or _force_plain or not _tc_operands(x, w_gate_up):
        return gemm_plain(x, w_gate_up, None, gated=True, gate_limit=limit)
    # Pairs of SMs (256 tokens x 128 features per tile, gate rows in one CTA and up rows in the other)
    # once their tiles fill most of the 74 pairs: measured 6 to 12 % faster from there on at the 0.5B,
    # 1.5B and 7B layer sizes (2,048 tokens: 31.7 against 33.7, 76 against 85, 349 against 385 us).
    T, inter = x.shape[0], w_gate_up.shape[0] // 2
    if -(-T // 256) * (-(-inter // 128)) >= 64:
        return gemm_tc2(x, w_gate_up, None, gated=True, gate_limit=limit)
    return gemm_tc(x, w_gate_up, None, gated=True, gate_limit=limit)


# Which kernel serves requests that bring several tokens: "auto" (tcgen05 for heads of 64 and of 128
# once a request brings more than 64 tokens, else mma.sync), "mma" or "tc05".
PREFILL_KERNEL = "auto"


# With 2 to 8 splits, and all CTAs of the launch resident at once, the decode kernel merges the splits
# itself: the splits of a (request, kv head) form a thread-block cluster and read one another's shared
# memory.  (With more CTAs than SMs the cluster launch measured slower than the merge kernel.)
# False: always the merge kernel.
CLUSTER_MERGE = True


def attention_tc_supported(head_dim: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= 128


def decode_shape(head_dim: int) -> tuple[int, int]:
    """(keys a decode CTA takes in one round of its warps, decode CTAs an SM holds) of the kernel
    built for this head size."""
    shape = _decode_shapes.get(head_dim)
    if shape is None:
        L = lib("attention_tc", {"LAB_HEAD_DIM": head_dim})
        shape = _decode_shapes[head_dim] = (int(L.lab_attention_decode_keys_per_round()),
                                            int(L.lab_attention_decode_ctas_per_sm()))
    return shape


_decode_shapes: dict[int, tuple[int, int]] = {}


def decode_splits(n_decode: int, n_kv: int, group: int, max_kv_len: int, keys_per_round: int = 128,
                  ctas_per_sm: int = 2) -> int:
    """How many ways the keys of a decoding request are split across CTAs.  A warp needs about
    two microseconds per tile (its instructions depend on one another), so for latency a
    CTA's warps should get one tile each: one round (128 keys at heads of 64) per CTA while all
    CTAs of the launch find room at once and the splits (8 at most) can merge inside their cluster;
    else two rounds per CTA, as far as the GPU has room for the CTAs (the reference splits 1..16
    ways, rust/engine/src/runner/model/qwen2/engine.rs:1597-1617)."""
    ctas = max(1, n_decode * n_kv * (-(-group // 16)))
    if CLUSTER_MERGE and max_kv_len <= 16 * keys_per_round:     # beyond that, more than 8 splits serve better
        fine = min(8, -(-max_kv_len // keys_per_round), sm_count() // ctas)
        if fine >= 2:
            return int(fine)
    room = max(1, (ctas_per_sm * sm_count()) // ctas)      # no second round of CTAs
    return int(max(1, min(room, -(-max_kv_len // (2 * keys_per_round)), 32)))


TC05_BIAS_MAX = 4096     # entries of a distance table the tcgen05 prefill kernel holds (its BIAS_MAX)


def attention_tc(q, cache_k, cache_v, q_start, kv_len, pos0, block_table, n_requests, q_lens, max_kv_len,
                 n_q, n_kv, head_dim, window, scale, out=None, splits=None, scratch=None, keep_first=0, sink=None,
                 dist_bias=None):
    """Tensor-core attention: the prefill kernel serves requests with several new tokens,
    the split-KV decode kernel those with one.  A negative `window` means chunks of that many positions.
    `keep_first`: beside a window, the first that many positions stay visible.  `sink`: 32-bit numbers, one per
    query head, that join the softmax's denominator as exp(sink) (a key with that unscaled score and no value).
    `dist_bias` [n_q, L] 32-bit: a number per head and distance query - key added to the scaled score, distances
    from L - 1 on sharing the last entry (the tcgen05 kernel keeps a head's table in shared memory, up to
    `TC05_BIAS_MAX` entries; longer tables run on the `mma.sync` prefill kernel)."""
    _on_gpu(q, cache_k, cache_v, q_start, kv_len, pos0, block_table, sink, dist_bias)
    assert dist_bias is None or (dist_bias.dtype == torch.float32 and dist_bias.dim() == 2 and
                                 dist_bias.shape[0] == n_q and dist_bias.is_contiguous())
    bias_len = dist_bias.shape[1] if dist_bias is not None else 0
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() >= n_q and sink.is_contiguous())
    keep_first = int(keep_first) if window > 0 else 0
    if q.dtype != torch.bfloat16 or not attention_tc_supported(head_dim):
        raise KernelError(f"attention_tc: bfloat16 and a head size multiple of 16 up to 128, got {q.dtype}, {head_dim}")
    tokens = q.shape[0]
    if out is None:
        out = torch.empty((tokens, n_q * head_dim), dtype=q.dtype, device=q.device)
    num_pages, kvh, page_size, d = cache_k.shape
    assert kvh == n_kv and d == head_dim and q.stride(1) == 1 and q.stride(0) % 8 == 0
    assert block_table.dim() == 2 and block_table.is_contiguous() and block_table.shape[0] >= n_requests
    L = lib("attention_tc", {"LAB_HEAD_DIM": head_dim})
    max_q = max(q_lens)
    n_decode = sum(1 for n in q_lens if n == 1)
    use_tc05 = PREFILL_KERNEL == "tc05" or (PREFILL_KERNEL == "auto" and max_q > 64)
    if max_q > 1 and use_tc05 and head_dim in (64, 128) and page_size >= 8 and page_size <= 128 and \
            page_size & (page_size - 1) == 0 and bias_len <= TC05_BIAS_MAX:
        # tcgen05 kernel: tiles of 128 query rows, scores and P V on the 5th-generation tensor cores
        L5 = lib("attention_tc05", {"LAB_HEAD_DIM": head_dim})
        _check(L5.lab_attention_prefill_tc05(
            _ptr(out), out.stride(0), _ptr(q), q.stride(0), tokens, _ptr(cache_k), _ptr(cache_v), _ptr(q_start),
            _ptr(kv_len), _ptr(pos0), _ptr(block_table), block_table.shape[1], n_requests, max_q, n_q, n_kv,
            page_size, num_pages, window, ctypes.c_float(scale), 2, keep_first, _ptr(sink), _ptr(dist_bias), bias_len,
            _stream()),
            "attention_prefill_tc05")
    elif max_q > 1:
        _check(L.lab_attention_prefill(_ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(cache_k), _ptr(cache_v),
                                       _ptr(q_start), _ptr(kv_len), _ptr(pos0), _ptr(block_table),
                                       block_table.shape[1], n_requests, max_q, n_q, n_kv, page_size, num_pages,
                                       window, ctypes.c_float(scale), 2, _ptr(sink), keep_first, _ptr(dist_bias),
                                       bias_len, _stream()),
               "attention_prefill")
    if n_decode:
        if splits is None:
            span = min(max_kv_len, abs(window) + keep_first) if window else max_kv_len     # a chunk reaches as far as a window
            splits = decode_splits(n_decode, n_kv, n_q // n_kv, span, *decode_shape(head_dim))
        ctas = n_decode * n_kv * (-(-(n_q // n_kv) // 16)) * splits
        in_cluster = CLUSTER_MERGE and 2 <= splits <= 8 and ctas <= sm_count()
        if splits > 1 and not in_cluster:
            need = n_requests * n_q * splits * (head_dim + 2)
            if scratch is None or scratch.numel() < need:
                scratch = torch.empty((need,), dtype=torch.float32, device=q.device)
        else:
            scratch = None
        _check(L.lab_attention_decode(_ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(cache_k), _ptr(cache_v),
                                      _ptr(q_start), _ptr(kv_len), _ptr(block_table), block_table.shape[1],
                                      n_requests, n_q, n_kv, page_size, num_pages, window, ctypes.c_float(scale),
                                      splits, _ptr(scratch), 1 if in_cluster else 0, keep_first, _ptr(sink),
                                      _ptr(dist_bias), bias_len, _stream()),
               "attention_decode",
               2 if splits > 1 and not in_cluster else 1)
    return out


def attention(q, cache_k, cache_v, ctx, group, n_q, n_kv, head_dim, window, scale, chunk=0, keep_first=0,
              sink_one=False, sink=None, dist_bias=None):
    """Causal attention of every row over its request's cached keys: all of them, the last `window`, or
    (with `chunk`) those of the row's own chunk of `chunk` positions, chunks counted from position 0.  The
    kernels take the mask as one number: a window as it is, a chunk as its negative.  `keep_first`: beside a
    window, the first that many positions of the sequence stay visible; `sink_one`: the softmax's denominator
    holds one more (a key with score 0 and no value); `sink` [n_q] 32-bit: it holds exp(sink[h]) more instead (a
    learned score of that key, unscaled); `dist_bias` [n_q, L] 32-bit: a number per head and distance query - key
    added to the scaled score, distances from L - 1 on sharing the last entry."""
    if sink is not None:
        sink_one = False
    if chunk:
        if window:
            raise KernelError("attention takes a window or a chunk, not both")
        window = -int(chunk)
    if keep_first and window <= 0:
        keep_first = 0          # kept first positions only matter beside a window
    if q.dtype == torch.bfloat16 and not _force_plain and attention_tc_supported(head_dim):
        # the denominator's extra one is a sink of 0 for every head
        return attention_tc(q, cache_k, cache_v, ctx.q_start, ctx.kv_len, ctx.pos0, group.block_table,
                            ctx.n_requests, ctx.q_lens, ctx.max_kv_len, n_q, n_kv, head_dim, window, scale,
                            keep_first=keep_first, dist_bias=dist_bias,
                            sink=sink if sink is not None else (_zero_sinks(q.device, n_q) if sink_one else None))
    return attention_plain(q, cache_k, cache_v, ctx.row_req, ctx.row_pos, group.block_table, n_q, n_kv, head_dim,
                           window, scale, keep_first=keep_first, sink_one=sink_one, sink=sink, dist_bias=dist_bias)


_zero_sink_cache: dict = {}


def _zero_sinks(device, n_q: int) -> torch.Tensor:
    """Zeros, one per query head (kept: a CUDA graph captured earlier still reads them)."""
    key = (str(device), n_q)
    t = _zero_sink_cache.get(key)
    if t is None:
        t = _zero_sink_cache[key] = torch.zeros((n_q,), dtype=torch.float32, device=device)
    return t


# ----------------------------------------------------------------------------------------
# Operators on a residual stream kept in 32-bit floats (csrc/kernels/stream32.cu).
# ----------------------------------------------------------------------------------------
def embed_norm(ids: torch.Tensor, table: torch.Tensor, weight: torch.Tensor, eps: float, offset: float) -> torch.Tensor:
    """32-bit rows table[id] / rms(table[id]) * (offset + weight)."""
    _on_gpu(ids, table, weight)
    tokens, (vocab, hidden) = ids.numel(), table.shape
    assert ids.dtype == torch.int32 and table.is_contiguous() and weight.dtype == table.dtype
    out = torch.empty((tokens, hidden), dtype=torch.float32, device=table.device)
    _check(lib("stream32").lab_embed_norm(_ptr(out), _ptr(table), _ptr(ids), _ptr(weight), tokens, hidden, vocab,
                                          ctypes.c_float(eps), ctypes.c_float(offset), dtype_code(table.dtype),
                                          _stream()), "embed_norm")
    return out


def norm_stream(x: torch.Tensor, eps: float, offset: float, weight_f32: torch.Tensor | None = None,
                weight: torch.Tensor | None = None, rows: torch.Tensor | None = None):
    """RMS norms of the rows of a 32-bit stream `x`, gain (offset + weight): with `weight_f32` a 32-bit
    result, with `weight` one rounded to the weight's storage type; both at once read x once.  With
    `rows`, output row i comes from x[rows[i]].  Returns (32-bit result or None, stored result or None)."""
    _on_gpu(x, weight_f32, weight, rows)
    n_in, hidden = x.shape
    n_out = n_in if rows is None else rows.numel()
    assert x.dtype == torch.float32 and x.is_contiguous() and (weight_f32 is not None or weight is not None)
    wdt = (weight if weight is not None else weight_f32).dtype
    assert weight_f32 is None or weight is None or weight_f32.dtype == weight.dtype
    out_a = torch.empty((n_out, hidden), dtype=torch.float32, device=x.device) if weight_f32 is not None else None
    out_b = torch.empty((n_out, hidden), dtype=wdt, device=x.device) if weight is not None else None
    _check(lib("stream32").lab_norm_stream(_ptr(out_a), _ptr(out_b), _ptr(x), _ptr(weight_f32), _ptr(weight), _ptr(rows),
                                           n_out, n_in, hidden, ctypes.c_float(eps), ctypes.c_float(offset),
                                           dtype_code(wdt), _stream()), "norm_stream")
    return out_a, out_b


def token_shift(normed: torch.Tensor, mix: torch.Tensor, kept: torch.Tensor, ctx, write: bool = True) -> torch.Tensor:
    """h[t] = n[t] + (n[t-1] - n[t]) * mix over the rows of each request, the row before a request's
    first row of this step taken from `kept` [slots, hidden] (zeros at position 0); `kept` then takes the
    request's last row.  `normed` is 32-bit; the result has mix's storage type."""
    _on_gpu(normed, mix, kept)
    tokens, hidden = normed.shape
    assert normed.dtype == torch.float32 and normed.is_contiguous() and kept.dtype == torch.float32
    assert kept.is_contiguous() and kept.shape[1] == hidden and mix.numel() == hidden
    out = torch.empty((tokens, hidden), dtype=mix.dtype, device=normed.device)
    _check(lib("stream32").lab_token_shift(_ptr(out), _ptr(normed), _ptr(mix), _ptr(kept), _ptr(ctx.row_req),
                                           _ptr(ctx.q_start), _ptr(ctx.pos0), _ptr(ctx.state_slot), tokens, hidden,
                                           kept.shape[0], int(write), dtype_code(mix.dtype), _stream()), "token_shift")
    return out


def stream_add(x: torch.Tensor, a: torch.Tensor, scale_a: torch.Tensor, b: torch.Tensor | None,
               scale_b: torch.Tensor | None, mult: float) -> torch.Tensor:
    """x += mult * (scale_a * a + scale_b * b) in place on the 32-bit stream; a and b are 32-bit products
    [tokens, hidden] or split-K partial products [splits, tokens, hidden] (summed in ascending order)."""
    _on_gpu(x, a, b, scale_a, scale_b)
    tokens, hidden = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous()

    def splits_of(t):
        assert t.dtype == torch.float32 and t.is_contiguous() and t.shape[-2:] == x.shape
        return t.shape[0] if t.dim() == 3 else 1

    sa = splits_of(a)
    sb = splits_of(b) if b is not None else 0
    assert scale_a.numel() == hidden and (b is None or (scale_b.numel() == hidden and scale_b.dtype == scale_a.dtype))
    _check(lib("stream32").lab_stream_add(_ptr(x), _ptr(a), sa, _ptr(b), sb, _ptr(scale_a), _ptr(scale_b),
                                          ctypes.c_longlong(tokens), hidden, ctypes.c_float(mult),
                                          dtype_code(scale_a.dtype), _stream()), "stream_add")
    return x


def stream_add_norm(x: torch.Tensor, a: torch.Tensor, scale_a: torch.Tensor, b: torch.Tensor | None,
                    scale_b: torch.Tensor | None, mult: float, eps: float, offset: float,
                    weight_f32: torch.Tensor | None = None, weight: torch.Tensor | None = None,
                    rows: torch.Tensor | None = None):
    """`stream_add` and `norm_stream` in one pass over the rows: x += mult * (scale_a * a + scale_b * b), then
    the norms of the sum.  With `rows` only those rows are formed and x is left as it is."""
    _on_gpu(x, a, b, scale_a, scale_b, weight_f32, weight, rows)
    n_in, hidden = x.shape
    n_out = n_in if rows is None else rows.numel()
    assert x.dtype == torch.float32 and x.is_contiguous() and (weight_f32 is not None or weight is not None)

    def splits_of(t):
        assert t.dtype == torch.float32 and t.is_contiguous() and t.shape[-2:] == x.shape
        return t.shape[0] if t.dim() == 3 else 1

    sa = splits_of(a)
    sb = splits_of(b) if b is not None else 0
    wdt = scale_a.dtype
    assert all(w is None or w.dtype == wdt for w in (scale_b, weight_f32, weight))
    out_a = torch.empty((n_out, hidden), dtype=torch.float32, device=x.device) if weight_f32 is not None else None
    out_b = torch.empty((n_out, hidden), dtype=wdt, device=x.device) if weight is not None else None
    _check(lib("stream32").lab_stream_add_norm(
        _ptr(out_a), _ptr(out_b), _ptr(x), _ptr(a), sa, _ptr(b), sb, _ptr(scale_a), _ptr(scale_b), ctypes.c_float(mult),
        _ptr(weight_f32), _ptr(weight), _ptr(rows), n_out, n_in, hidden, ctypes.c_float(eps), ctypes.c_float(offset),
        dtype_code(wdt), _stream()), "stream_add_norm")
    return out_a, out_b


def stream_concat(x: torch.Tensor, x0: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """[x ; x0] row by row, rounded to `dtype`, for a projection that reads both."""
    _on_gpu(x, x0)
    tokens, hidden = x.shape
    assert x.dtype == torch.float32 and x0.dtype == torch.float32 and x.is_contiguous() and x0.is_contiguous()
    assert x0.shape == x.shape
    out = torch.empty((tokens, 2 * hidden), dtype=dtype, device=x.device)
    _check(lib("stream32").lab_stream_concat(_ptr(out), _ptr(x), _ptr(x0), ctypes.c_longlong(tokens), hidden,
                                             dtype_code(dtype), _stream()), "stream_concat")
    return out


def softcap(logits: torch.Tensor, cap: float) -> torch.Tensor:
    """logits <- cap * tanh(logits / cap), in place on 32-bit logits."""
    _on_gpu(logits)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    _check(lib("stream32").lab_softcap(_ptr(logits), ctypes.c_longlong(logits.numel()), ctypes.c_float(cap), _stream()),
           "softcap")
    return logits


# ----------------------------------------------------------------------------------------
# Generalized delta rule (csrc/kernels/delta_rule.cu, built per head size).
# ----------------------------------------------------------------------------------------
def delta_rule_supported(head_dim: int) -> bool:
    return 4 <= head_dim <= 256


def tanh_cast(x: torch.Tensor, dtype: torch.dtype, head_dim: int = 64) -> torch.Tensor:
    """tanh of a 32-bit column slice [tokens, n], rounded to `dtype` and made contiguous (`head_dim`
    names the build of the delta rule's library to take it from)."""
    _on_gpu(x)
    tokens, n = x.shape
    assert x.dtype == torch.float32 and x.stride(1) == 1
    out = torch.empty((tokens, n), dtype=dtype, device=x.device)
    _check(lib("delta_rule", {"LAB_HEAD_DIM": head_dim}).lab_tanh_cast(_ptr(out), _ptr(x), ctypes.c_longlong(tokens), n,
                                                                 x.stride(0), dtype_code(dtype), _stream()),
           "tanh_cast")
    return out


def delta_rule(proj: torch.Tensor, decay_pre: torch.Tensor, decay_bias: torch.Tensor, rate_bias: torch.Tensor,
               norm_weight: torch.Tensor, state: torch.Tensor, ctx, heads: int, head_dim: int, eps: float,
               decay_rate: float, write: bool = True) -> torch.Tensor:
    """The recurrence over each request's rows.  `proj` [tokens, >= 5 * heads * head_dim] 32-bit holds
    r, k, v, the gate's and the removal rate's pre-activations side by side; `decay_pre` [tokens,
    heads * head_dim] the decay's; `state` [slots, heads, head_dim, head_dim] 32-bit is read and (with
    `write`) left advanced.  Returns the normalised, gated output in the biases' storage type."""
    _on_gpu(proj, decay_pre, decay_bias, rate_bias, norm_weight, state)
    tokens, hd = proj.shape[0], heads * head_dim
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[1] >= 5 * hd
    assert decay_pre.dtype == torch.float32 and decay_pre.stride(1) == 1 and decay_pre.shape == (tokens, hd)
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (heads, head_dim, head_dim)
    dt = decay_bias.dtype
    assert rate_bias.dtype == dt and norm_weight.dtype == dt
    assert decay_bias.numel() == hd and rate_bias.numel() == hd and norm_weight.numel() == hd
    if not delta_rule_supported(head_dim):
        raise KernelError(f"delta_rule: head size {head_dim} outside 4..256")
    out = torch.empty((tokens, hd), dtype=dt, device=proj.device)
    L = lib("delta_rule", {"LAB_HEAD_DIM": head_dim})
    L.lab_delta_rule_scratch.restype = ctypes.c_longlong
    raw = torch.empty((int(L.lab_delta_rule_scratch(tokens, heads)),), dtype=torch.float32, device=proj.device)
    base, esz = proj.data_ptr(), 4

    def col(i):
        return ctypes.c_void_p(base + esz * i * hd)

    _check(L.lab_delta_rule(_ptr(out), _ptr(raw), col(0), col(1), col(2), col(3), col(4), proj.stride(0),
                            _ptr(decay_pre), decay_pre.stride(0), _ptr(decay_bias), _ptr(rate_bias), _ptr(norm_weight),
                            _ptr(state), _ptr(ctx.q_start), _ptr(ctx.state_slot), tokens, ctx.n_requests, heads,
                            state.shape[0], int(write), ctypes.c_float(eps), ctypes.c_float(decay_rate),
                            dtype_code(dt), _stream()), "delta_rule", 3)
    return out


# ----------------------------------------------------------------------------------------
# Attention over a paged cache of latents (csrc/kernels/latent_attention.cu).
# ----------------------------------------------------------------------------------------
def latent_prep(proj: torch.Tensor, q_rank: int, kv_rank: int, rot_dim: int, w_q: torch.Tensor, w_c: torch.Tensor,
                positions: torch.Tensor, inv_freq: torch.Tensor, rot_dims: int, slots: torch.Tensor | None,
                cache: torch.Tensor | None, eps: float, pairs: bool = False) -> torch.Tensor:
    """From the 32-bit low-rank projections of a step's rows [tokens, q_rank + kv_rank + rot_dim]: the
    normalised query latent (returned, in the weights' storage type; None where q_rank is 0: queries
    projected directly), `pairs`: the rotation turns neighbouring entries (2i, 2i + 1) instead of (i, i + half);
    and, into each row's cache slot,
    the normalised key/value latent followed by the rotated shared key part (`cache` None: no write)."""
    _on_gpu(proj, w_q, w_c, positions, inv_freq, slots, cache)
    tokens = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[1] == q_rank + kv_rank + rot_dim
    assert w_c.numel() == kv_rank and ((q_rank == 0 and w_q is None) or (w_q.numel() == q_rank and w_q.dtype == w_c.dtype))
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dims // 2 and rot_dims <= rot_dim
    n_slots = 0
    if cache is not None:
        assert cache.is_contiguous() and cache.shape[2] == kv_rank + rot_dim and cache.dtype == w_c.dtype
        assert slots is not None and slots.dtype == torch.int32
        n_slots = cache.shape[0] * cache.shape[1]
    cq = torch.empty((tokens, q_rank), dtype=w_c.dtype, device=proj.device) if q_rank else None
    _check(lib("latent_attention").lab_latent_prep(
        _ptr(cq), _ptr(cache), _ptr(proj), proj.stride(0), q_rank, kv_rank, rot_dim, _ptr(w_q), _ptr(w_c),
        _ptr(positions), _ptr(inv_freq), rot_dims, _ptr(slots), ctypes.c_longlong(n_slots), tokens,
        ctypes.c_float(eps), int(bool(pairs)), dtype_code(w_c.dtype), _stream()), "latent_prep")
    return cq


def latent_q_rope(q: torch.Tensor, q_cat: torch.Tensor | None, heads: int, dim: int, rot_dim: int, kv_rank: int,
                  positions: torch.Tensor, inv_freq: torch.Tensor, rot_dims: int, in_place: bool = False,
                  pairs: bool = False) -> None:
    """Rotates entries [dim, dim + rot_dim) of every head of q [tokens, heads * q_head] (q_head >= dim + rot_dim:
    a head may end in padding) into columns [kv_rank, kv_rank + rot_dim) of each head of the 32-bit q_cat
    [tokens, heads, kv_rank + rot_dim]; with `in_place` also into q itself (q_cat may then be None)."""
    _on_gpu(q, q_cat, positions, inv_freq)
    tokens = q.shape[0]
    q_head = q.shape[1] // heads
    assert q.is_contiguous() and q.shape[1] == heads * q_head and q_head >= dim + rot_dim
    assert q_cat is None or (q_cat.dtype == torch.float32 and q_cat.is_contiguous()
                             and q_cat.shape == (tokens, heads, kv_rank + rot_dim))
    assert q_cat is not None or in_place
    _check(lib("latent_attention").lab_latent_q_rope(_ptr(q_cat), _ptr(q), tokens, heads, dim, rot_dim, kv_rank, q_head,
                                                     _ptr(positions), _ptr(inv_freq), rot_dims, int(in_place),
                                                     int(bool(pairs)), dtype_code(q.dtype), _stream()), "latent_q_rope")


def latent_attention(q_cat: torch.Tensor, cache: torch.Tensor, sink: torch.Tensor | None, ctx, group, heads: int,
                     kv_rank: int, window: int, scale: float, below: int = 0) -> torch.Tensor:
    """Every row's heads over the latents of its request's pages: scores q_cat . [c ; kr] * scale,
    softmax in 32-bit whose denominator also holds exp(sink) per head, output the weighted sum of the
    latents c, [tokens, heads * kv_rank] in the cache's storage type.  `below` > 0: only the rows of
    requests that bring fewer rows than that are computed (the others' rows are left as they are)."""
    _on_gpu(q_cat, cache, sink)
    tokens, width = q_cat.shape[0], q_cat.shape[2]
    num_pages, page_size, w = cache.shape
    assert w == width and cache.is_contiguous() and q_cat.dtype == torch.float32 and q_cat.is_contiguous()
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == heads)
    L = lib("latent_attention")
    max_q = min(ctx.max_q_len, below - 1) if below > 0 else ctx.max_q_len
    if L.lab_latent_attention_rows(heads, kv_rank, width, max_q) <= 0:
        raise KernelError(f"latent_attention: {heads} heads of width {width} do not fit shared memory")
    out = torch.empty((tokens, heads * kv_rank), dtype=cache.dtype, device=cache.device)
    table = group.block_table
    splits, part = 1, None
    if max_q == 1:
        # single tokens: the keys' tiles (32 keys each) of a request are shared out over CTAs while the launch
        # stays within two rounds of the SMs, two tiles a share at least; a merge kernel sums the shares
        span = min(ctx.max_kv_len, window) if window > 0 else ctx.max_kv_len
        ctas = ctx.n_requests * -(-heads // max(1, L.lab_latent_attention_heads(heads, kv_rank, width, 1)))
        splits = int(max(1, min(-(-span // 64), (2 * sm_count()) // max(ctas, 1), 64)))
        if splits > 1:
            part = torch.empty((ctx.n_requests * heads * splits * (kv_rank + 2),), dtype=torch.float32,
                               device=cache.device)
    _check(L.lab_latent_attention(_ptr(out), _ptr(q_cat), _ptr(cache), _ptr(sink), _ptr(ctx.q_start), _ptr(ctx.pos0),
                                  _ptr(ctx.kv_len), _ptr(table), table.shape[1], ctx.n_requests, max_q, heads, kv_rank, width,
                                  page_size, num_pages, window, ctypes.c_float(scale), int(below), splits, _ptr(part),
                                  dtype_code(cache.dtype), _stream()), "latent_attention", 2 if splits > 1 else 1)
    return out


_latent_pools: dict = {}


def latent_plain_form_supported(dtype, dim: int, rot_dim: int, vdim: int) -> bool:
    """Whether prompts' portions of a latent attention can run on the tensor-core attention kernel with keys
    and values projected up for the step: bfloat16, and heads (key = dim + rot_dim, value = vdim, the
    larger one rounded up to a multiple of 16) within the kernel's 128."""
    return dtype == torch.bfloat16 and not _force_plain and latent_head_size(dim, rot_dim, vdim) <= 128


def latent_head_size(dim: int, rot_dim: int, vdim: int) -> int:
    return (max(dim + rot_dim, vdim) + 15) // 16 * 16


def latent_attention_plain_form(q: torch.Tensor, cache: torch.Tensor, w_up: torch.Tensor, sink: torch.Tensor | None,
                                ctx, group, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, window: int,
                                scale: float, at_least: int, out: torch.Tensor) -> torch.Tensor:
    """The rows of requests that bring `at_least` rows or more, in the plain form: for every key such a
    request's rows can see, the head's key [W_uk c ; kr] and value W_uv c are projected up from the cached
    latent (`w_up` = [W_uk ; W_uv], one product) into scratch pools numbered like the cache's pages; then the
    tensor-core attention kernel of prompts runs over them with the step's own block table, window and
    sink.  q [tokens, heads * HD] holds rotated queries (HD = `latent_head_size`, padding zero); the heads'
    outputs go to `out` [tokens, heads * HD] (value entries first, padding zero)."""
    _on_gpu(q, cache, w_up, sink, out)
    hd = latent_head_size(dim, rot_dim, vdim)
    num_pages, page_size, width = cache.shape
    tokens = q.shape[0]
    assert q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and q.shape == (tokens, heads * hd)
    assert out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous() and q.is_contiguous()
    assert w_up.shape == (heads * (dim + vdim), kv_rank) and w_up.is_contiguous() and width == kv_rank + rot_dim
    meta, at, most = [], 0, 0
    for r, (n, kv) in enumerate(zip(ctx.q_lens, ctx.kv_lens)):
        if n < at_least:
            continue
        lo = max(0, kv - n - window + 1) if window > 0 else 0
        meta += [r, lo, kv - lo, at]
        at += kv - lo
        most = max(most, kv - lo)
    if not meta:
        return out
    key = (str(q.device), num_pages, heads, page_size, hd)
    pools = _latent_pools.get(key)
    if pools is None:
        _latent_pools.clear()       # one engine's pools at a time
        pools = _latent_pools[key] = (torch.zeros((num_pages, heads, page_size, hd), dtype=q.dtype, device=q.device),
                                      torch.zeros((num_pages, heads, page_size, hd), dtype=q.dtype, device=q.device))
    meta_t = torch.tensor(meta, dtype=torch.int32).to(q.device, non_blocking=True)
    compact = torch.empty((at, kv_rank), dtype=q.dtype, device=q.device)
    slot_of = torch.empty((at,), dtype=torch.int32, device=q.device)
    L = lib("latent_attention")
    table = group.block_table
    _check(L.lab_latent_gather(_ptr(compact), _ptr(slot_of), _ptr(cache), _ptr(meta_t), len(meta) // 4, most,
                               _ptr(table), table.shape[1], kv_rank, width, page_size, num_pages, _stream()),
           "latent_gather")
    projected = linear(compact, w_up, None)
    _check(L.lab_latent_scatter(_ptr(pools[0]), _ptr(pools[1]), _ptr(projected), _ptr(slot_of), _ptr(cache), at, heads,
                                dim, rot_dim, vdim, kv_rank, hd, page_size, _stream()), "latent_scatter")
    LA = lib("attention_tc", {"LAB_HEAD_DIM": hd})
    _check(LA.lab_attention_prefill(_ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(pools[0]), _ptr(pools[1]),
                                    _ptr(ctx.q_start), _ptr(ctx.kv_len), _ptr(ctx.pos0), _ptr(table), table.shape[1],
                                    ctx.n_requests, ctx.max_q_len, heads, heads, page_size, num_pages, window,
                                    ctypes.c_float(scale), int(at_least), _ptr(sink), 0, None, 0, _stream()), "attention_prefill")
    return out


# ----------------------------------------------------------------------------------------
# A 32-bit stream with learned positions and normed sublayer outputs (csrc/kernels/stream32.cu).
# ----------------------------------------------------------------------------------------
def embed_position(ids: torch.Tensor, positions: torch.Tensor | None, table: torch.Tensor,
                   pos_table: torch.Tensor | None, scale: float = 1.0) -> torch.Tensor:
    """32-bit rows table[id] * scale + pos_table[position]; without a position table, table[id] * scale alone."""
    _on_gpu(ids, positions, table, pos_table)
    tokens, (vocab, hidden) = ids.numel(), table.shape
    assert ids.dtype == torch.int32 and table.is_contiguous()
    if pos_table is not None:
        assert positions.dtype == torch.int32 and positions.numel() == tokens
        assert pos_table.is_contiguous() and pos_table.shape[1] == hidden and pos_table.dtype == table.dtype
    out = torch.empty((tokens, hidden), dtype=torch.float32, device=table.device)
    _check(lib("stream32").lab_embed_position(_ptr(out), _ptr(table), _ptr(pos_table), _ptr(ids),
                                              _ptr(positions if pos_table is not None else None), tokens, hidden,
                                              vocab, pos_table.shape[0] if pos_table is not None else 0,
                                              ctypes.c_float(scale), dtype_code(table.dtype), _stream()), "embed_position")
    return out


def stream_norm_add(x: torch.Tensor, a: torch.Tensor, weight: torch.Tensor, eps: float,
                    bias: torch.Tensor | None = None, copy: bool = False,
                    next_weight: torch.Tensor | None = None) -> torch.Tensor | None:
    """x += rmsnorm(a + bias) * weight in place on the 32-bit stream; `a` is a 32-bit product [tokens, hidden]
    or split-K partial products [splits, tokens, hidden] (summed in ascending order).  With `copy`, returns
    the new rows of x rounded to the weight's storage type; with `next_weight`, returns rmsnorm(new x) *
    next_weight instead (the norm that opens the next sublayer), rounded likewise."""
    _on_gpu(x, a, weight, bias, next_weight)
    copy = copy or next_weight is not None
    assert next_weight is None or (next_weight.dtype == weight.dtype and next_weight.numel() == x.shape[1])
    tokens, hidden = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and a.dtype == torch.float32 and a.is_contiguous()
    assert a.shape[-2:] == x.shape and weight.numel() == hidden and (bias is None or bias.dtype == weight.dtype)
    splits = a.shape[0] if a.dim() == 3 else 1
    rounded = torch.empty((tokens, hidden), dtype=weight.dtype, device=x.device) if copy else None
    _check(lib("stream32").lab_stream_norm_add(_ptr(x), _ptr(rounded), _ptr(a), splits, _ptr(bias), _ptr(weight), tokens,
                                               hidden, ctypes.c_float(eps), _ptr(next_weight),
                                               dtype_code(weight.dtype), _stream()),
           "stream_norm_add")
    return rounded


def stream_round(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The 32-bit stream rounded to `dtype` (the stream itself where that is 32-bit)."""
    if dtype == torch.float32:
        return x
    _on_gpu(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _check(lib("stream32").lab_stream_round(_ptr(out), _ptr(x), ctypes.c_longlong(x.numel()), dtype_code(dtype), _stream()),
           "stream_round")
    return out


def weighted_sum(a: torch.Tensor, ca: float, b: torch.Tensor, cb: float) -> torch.Tensor:
    """ca * a + cb * b over 32-bit products [tokens, hidden] or split-K partial products [splits, tokens, hidden]."""
    _on_gpu(a, b)
    assert a.dtype == torch.float32 and b.dtype == torch.float32 and a.is_contiguous() and b.is_contiguous()
    assert a.shape[-2:] == b.shape[-2:]
    out = torch.empty(a.shape[-2:], dtype=torch.float32, device=a.device)
    _check(lib("stream32").lab_weighted_sum(_ptr(out), _ptr(a), a.shape[0] if a.dim() == 3 else 1, _ptr(b),
                                            b.shape[0] if b.dim() == 3 else 1, ctypes.c_longlong(out.numel()),
                                            ctypes.c_float(ca), ctypes.c_float(cb), _stream()), "weighted_sum")
    return out


# ----------------------------------------------------------------------------------------
# Attention with norms over the whole q and k projections and a gate (csrc/kernels/norm_attention.cu).
# ----------------------------------------------------------------------------------------
def padded_head(dim: int, vdim: int) -> int:
    """The width heads of `dim` keys and `vdim` values are stored at: the larger one rounded up to a multiple
    of 16 (the tensor-core attention's step)."""
    return (max(dim, vdim) + 15) // 16 * 16


def qk_norm_store(proj: torch.Tensor, bias, w_q: torch.Tensor, w_k, slots, cache_k, cache_v, n_q: int, n_kv: int,
                  dim: int, vdim: int, head: int, eps: float, has_kv: bool = True) -> torch.Tensor:
    """From the 32-bit fused projection `proj` [tokens, >= q + k + v columns] (or split-K partial products
    [splits, tokens, ...]) and an optional bias over those columns: q and k RMS-normed over their whole
    projections with the weights `w_q`, `w_k`; q returned [tokens, n_q * head] in the weights' storage type,
    heads padded with zeros to `head` entries; k and v written the same way into their cache slots
    (`cache_k` None: nothing is written).  `has_kv` False: the projection holds q only."""
    _on_gpu(proj, bias, w_q, w_k, slots, cache_k, cache_v)
    splits = proj.shape[0] if proj.dim() == 3 else 1
    tokens, ld = proj.shape[-2], proj.stride(-2)       # a column slice of a wider product will do
    assert proj.dtype == torch.float32 and proj.stride(-1) == 1 and (splits == 1 or proj.stride(0) == tokens * ld)
    need = n_q * dim + (n_kv * (dim + vdim) if has_kv else 0)
    assert proj.shape[-1] >= need and w_q.numel() == n_q * dim and (not has_kv or w_k.numel() == n_kv * dim)
    assert bias is None or (bias.numel() >= need and bias.dtype == w_q.dtype)
    dt = w_q.dtype
    page_size = num_pages = 0
    if cache_k is not None:
        num_pages, kvh, page_size, d = cache_k.shape
        assert has_kv and kvh == n_kv and d == head and cache_k.is_contiguous() and cache_v.is_contiguous()
        assert cache_v.shape == cache_k.shape and cache_k.dtype == dt and slots is not None and slots.dtype == torch.int32
    q = torch.empty((tokens, n_q * head), dtype=dt, device=proj.device)
    _check(lib("norm_attention").lab_qk_norm_store(
        _ptr(q), q.stride(0), _ptr(cache_k), _ptr(cache_v), _ptr(proj), splits, ld, _ptr(bias), _ptr(w_q), _ptr(w_k),
        _ptr(slots), tokens, n_q, n_kv, dim, vdim, head, page_size, num_pages, int(has_kv), ctypes.c_float(eps),
        dtype_code(dt), _stream()), "qk_norm_store")
    return q


def head_gate(attn: torch.Tensor, proj: torch.Tensor, gate_at: int, per_head: bool, n_q: int, vdim: int, head: int,
              mult: float = 1.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[t, h * vdim + i] = attn[t, h * head + i] * sigmoid(g) * mult with g = proj[t, gate_at + h] (`per_head`)
    or proj[t, gate_at + h * vdim + i]; `proj` 32-bit, whole or split-K partial products.  `out` may be a
    column slice of a wider buffer."""
    _on_gpu(attn, proj, out)
    splits = proj.shape[0] if proj.dim() == 3 else 1
    tokens, ld = proj.shape[-2], proj.stride(-2)
    assert proj.dtype == torch.float32 and proj.stride(-1) == 1 and (splits == 1 or proj.stride(0) == tokens * ld)
    assert attn.stride(1) == 1 and attn.shape[0] == tokens
    assert proj.shape[-1] >= gate_at + (n_q if per_head else n_q * vdim)
    if out is None:
        out = torch.empty((tokens, n_q * vdim), dtype=attn.dtype, device=attn.device)
    assert out.dtype == attn.dtype and out.stride(1) == 1 and out.shape == (tokens, n_q * vdim)
    _check(lib("norm_attention").lab_head_gate(_ptr(out), out.stride(0), _ptr(attn), attn.stride(0), _ptr(proj), splits, ld,
                                               gate_at, int(per_head), tokens, n_q, vdim, head, ctypes.c_float(mult),
                                               dtype_code(attn.dtype), _stream()), "head_gate")
    return out


# ----------------------------------------------------------------------------------------
# Recurrent mixers with a scalar decay (csrc/kernels/linear_state.cu).
# ----------------------------------------------------------------------------------------
def decay_scan_supported(keys: int) -> bool:
    return 1 <= keys <= 256


def decay_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, ctx, heads: int, groups: int,
               keys: int, vdim: int, a_head: torch.Tensor | None = None, a_tok: torch.Tensor | None = None,
               s_tok: torch.Tensor | None = None, silu: bool = False, write: bool = True) -> torch.Tensor:
    """Per request and head, over the step's rows in order: S <- a S + (s k) v^T, o = S^T q, with S
    [keys, vdim] read from and (with `write`) left in `state` [slots, heads, keys, vdim].  q and k are 32-bit
    column slices [tokens, groups * keys] of one tensor (same row stride), v [tokens, heads * vdim]; `a_head`
    [heads] a fixed decay per head, or `a_tok`/`s_tok` [tokens, heads] per token; `silu`: q, k and v pass a
    SiLU first.  Returns o [tokens, heads * vdim] in 32-bit."""
    _on_gpu(q, k, v, state, a_head, a_tok, s_tok)
    tokens = v.shape[0]
    for t in (q, k, v):
        assert t.dtype == torch.float32 and t.stride(1) == 1 and t.shape[0] == tokens
    assert q.stride(0) == k.stride(0) and q.shape[1] == groups * keys and v.shape[1] == heads * vdim
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (heads, keys, vdim)
    assert (a_head is None) != (a_tok is None)
    ld_a = 0
    if a_tok is not None:
        assert a_tok.dtype == torch.float32 and a_tok.shape == (tokens, heads) and a_tok.stride(1) == 1
        assert s_tok is None or (s_tok.dtype == torch.float32 and s_tok.shape == (tokens, heads)
                                 and s_tok.stride(0) == a_tok.stride(0))
        ld_a = a_tok.stride(0)
    else:
        assert a_head.dtype == torch.float32 and a_head.numel() == heads and s_tok is None
    if not decay_scan_supported(keys):
        raise KernelError(f"decay_scan: {keys} key channels are outside what the recurrence kernel takes (1..256)")
    out = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=v.device)
    # Columns of the state per CTA.  Over a portion of a prompt the walk is one dependent chain per request and
    # head whatever the slice, and wide slices stage the keys and queries fewer times.  A step of single tokens
    # only reads and writes the state: narrow slices when it has few (request, head) pairs, so that more SMs work.
    pairs = ctx.n_requests * heads
    if ctx.max_q_len > 1:
        vs = 32
    else:
        vs = 32 if pairs * -(-vdim // 32) >= sm_count() else (16 if pairs * -(-vdim // 16) >= sm_count() else 8)
    vs = min(vs, max(8, 1 << (vdim - 1).bit_length()))
    _check(lib("linear_state").lab_decay_scan(
        _ptr(out), out.stride(0), _ptr(q), _ptr(k), q.stride(0), _ptr(v), v.stride(0), _ptr(a_tok), _ptr(s_tok), ld_a,
        _ptr(a_head), _ptr(state), _ptr(ctx.q_start), _ptr(ctx.state_slot), ctx.n_requests, state.shape[0], heads, groups,
        keys, vdim, int(silu), int(write), vs, _stream()), "decay_scan")
    return out


def ssm_prepare(proj: torch.Tensor, conv_at: int, dt_at: int, channels: int, taps: int, heads: int,
                taps_w: torch.Tensor, taps_b: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor,
                kept: torch.Tensor, ctx, write: bool = True):
    """From the 32-bit input projection `proj` of a state-space mixer: columns [conv_at, conv_at + channels)
    pass the causal convolution per channel (`taps_w` [channels, taps], last tap on the row itself; the
    inputs before a request's first row of the step come from `kept` [slots, taps - 1, channels], which with
    `write` then takes the request's last inputs) with bias and SiLU; columns [dt_at, dt_at + heads) give
    dt = softplus(. + dt_bias) and the decay exp(-exp(a_log) * dt).  Returns (convolved, dt, decay), 32-bit."""
    _on_gpu(proj, taps_w, taps_b, dt_bias, a_log, kept)
    tokens, ld = proj.shape[0], proj.stride(0)
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[1] >= max(conv_at + channels, dt_at + heads)
    assert taps_w.shape == (channels, taps) and taps_w.is_contiguous() and taps_b.numel() == channels
    assert dt_bias.numel() == heads and a_log.numel() == heads
    assert all(t.dtype == taps_w.dtype for t in (taps_b, dt_bias, a_log))
    assert kept.dtype == torch.float32 and kept.is_contiguous() and kept.shape[1:] == (max(taps - 1, 0), channels)
    conv = torch.empty((tokens, channels), dtype=torch.float32, device=proj.device)
    dt = torch.empty((tokens, heads), dtype=torch.float32, device=proj.device)
    decay = torch.empty((tokens, heads), dtype=torch.float32, device=proj.device)
    _check(lib("linear_state").lab_ssm_prepare(
        _ptr(conv), _ptr(dt), _ptr(decay), _ptr(proj), ld, conv_at, dt_at, channels, taps, heads, _ptr(taps_w),
        _ptr(taps_b), _ptr(dt_bias), _ptr(a_log), _ptr(kept), _ptr(ctx.row_req), _ptr(ctx.q_start), _ptr(ctx.state_slot),
        tokens, ctx.n_requests, kept.shape[0], int(write), dtype_code(taps_w.dtype), _stream()), "ssm_prepare",
        2 if write and taps > 1 else 1)
    return conv, dt, decay


def gated_norm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, parts: int = 1,
               gate_first: bool = False, skip: torch.Tensor | None = None, x: torch.Tensor | None = None,
               head_size: int = 1, mult: float = 1.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """The heads' outputs `o` [tokens, width] (32-bit; + skip[head] * x), gated and RMS-normed in `parts` equal
    parts with `weight`: `gate_first`, y * silu(gate) then the norm; else the norm then * sigmoid(gate).  `gate`
    and `x` are 32-bit column slices.  The result, times `mult`, is rounded to the weight's storage type."""
    _on_gpu(o, gate, weight, skip, x, out)
    tokens, width = o.shape
    assert o.dtype == torch.float32 and o.stride(1) == 1 and gate.dtype == torch.float32 and gate.stride(1) == 1
    assert gate.shape == o.shape and weight.numel() == width and width % parts == 0
    assert (skip is None) == (x is None)
    if skip is not None:
        assert x.dtype == torch.float32 and x.stride(1) == 1 and x.shape == o.shape and skip.dtype == weight.dtype
        assert skip.numel() * head_size == width
    if out is None:
        out = torch.empty((tokens, width), dtype=weight.dtype, device=o.device)
    assert out.dtype == weight.dtype and out.stride(1) == 1 and out.shape == (tokens, width)
    _check(lib("linear_state").lab_gated_norm(
        _ptr(out), out.stride(0), _ptr(o), o.stride(0), _ptr(x), x.stride(0) if x is not None else 0, _ptr(skip),
        head_size, _ptr(gate), gate.stride(0), _ptr(weight), tokens, width, parts, int(gate_first), ctypes.c_float(eps),
        ctypes.c_float(mult), dtype_code(weight.dtype), _stream()), "gated_norm")
    return out


def gelu_tanh_(x: torch.Tensor) -> torch.Tensor:
    """x <- 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) in place (32-bit arithmetic, one rounding)."""
    _on_gpu(x)
    assert x.is_contiguous()
    _check(lib("rowwise").lab_gelu_tanh(_ptr(x), ctypes.c_longlong(x.numel()), dtype_code(x.dtype), _stream()), "gelu_tanh")
    return x


# ----------------------------------------------------------------------------------------
# Rotation of neighbouring pairs with the paged store (csrc/kernels/rope_pairs.cu).
# ----------------------------------------------------------------------------------------
def rope_pairs_store(proj: torch.Tensor, bias, positions: torch.Tensor, inv_freq: torch.Tensor, rot_dims: int, slots,
                     cache_k, cache_v, n_q: int, n_kv: int, dim: int, vdim: int, head: int, k_at: int, v_at: int,
                     dtype: torch.dtype) -> torch.Tensor:
    """From the 32-bit projection of a step's rows (whole [tokens, width] or split-K partial products
    [splits, tokens, width]; q heads first, key heads from column k_at, value heads from v_at, which may equal
    k_at: the values are then the keys before their rotation): bias added, the first `rot_dims` entries of every
    q and k head turned pair by pair (entries 2i and 2i + 1 by position * inv_freq[i]), q returned in `dtype`
    [tokens, n_q * head] (zeros beyond `dim`), k and v written to the rows' slots (`slots` None: no write)."""
    _on_gpu(proj, bias, positions, inv_freq, slots, cache_k, cache_v)
    splits = proj.shape[0] if proj.dim() == 3 else 1
    tokens, ld = proj.shape[-2], proj.shape[-1]
    assert proj.dtype == torch.float32 and proj.is_contiguous()
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() >= rot_dims // 2
    assert bias is None or bias.dtype == dtype
    write = slots is not None
    n_slots = page_size = 0
    if write:
        assert cache_k.shape == cache_v.shape and cache_k.shape[1] == n_kv and cache_k.shape[3] == head
        assert cache_k.dtype == dtype and cache_k.is_contiguous() and cache_v.is_contiguous()
        page_size = cache_k.shape[2]
        n_slots = cache_k.shape[0] * page_size
    q = torch.empty((tokens, n_q * head), dtype=dtype, device=proj.device)
    _check(lib("rope_pairs").lab_rope_pairs_store(
        _ptr(q), _ptr(cache_k if write else None), _ptr(cache_v if write else None), _ptr(proj), splits,
        ctypes.c_longlong(tokens * ld), ld, k_at, v_at, _ptr(bias), _ptr(positions), _ptr(inv_freq), rot_dims,
        _ptr(slots), ctypes.c_longlong(n_slots), tokens, n_q, n_kv, dim, vdim, head, max(page_size, 1),
        dtype_code(dtype), _stream()), "rope_pairs_store")
    return q


# ----------------------------------------------------------------------------------------
# Selective scan (csrc/kernels/selective_scan.cu).
# ----------------------------------------------------------------------------------------
SELECTIVE_SCAN_MAX_STATE = 256


def conv_silu(proj: torch.Tensor, conv_at: int, channels: int, taps: int, w: torch.Tensor, b: torch.Tensor,
              kept: torch.Tensor, ctx, write: bool = True):
    """silu(causal convolution) of columns [conv_at, conv_at + channels) of the 32-bit `proj` over each request's
    last `taps` inputs (w [channels, taps], the last column on the row itself; bias b); `kept`
    [slots, taps - 1, channels] holds every request's last inputs between steps and is brought up to date when
    `write`.  Returns (32-bit result, the same rounded to the weights' type: the same tensor in a 32-bit engine)."""
    _on_gpu(proj, w, b, kept)
    tokens = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and w.is_contiguous() and w.shape == (channels, taps)
    assert kept.dtype == torch.float32 and kept.is_contiguous() and tuple(kept.shape[1:]) == (max(taps - 1, 0), channels)
    out32 = torch.empty((tokens, channels), dtype=torch.float32, device=proj.device)
    out_t = out32 if w.dtype == torch.float32 else torch.empty((tokens, channels), dtype=w.dtype, device=proj.device)
    _check(lib("selective_scan").lab_conv_silu(
        _ptr(out32), _ptr(None if out_t is out32 else out_t), _ptr(proj), proj.stride(0), conv_at, channels, taps,
        _ptr(w), _ptr(b), _ptr(kept), _ptr(ctx.row_req), _ptr(ctx.q_start), _ptr(ctx.state_slot), tokens, ctx.n_requests,
        kept.shape[0], int(write), dtype_code(w.dtype), _stream()), "conv_silu", 2 if write and taps > 1 else 1)
    return out32, out_t


def selective_scan(x: torch.Tensor, dt_pre: torch.Tensor, bc: torch.Tensor, b_at: int, c_at: int, z: torch.Tensor,
                   a_log: torch.Tensor, skip: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor, ctx,
                   write: bool = True) -> torch.Tensor:
    """The walk of a state-space mixer with a decay per channel and state entry: 32-bit x, dt_pre, z
    [tokens, channels] (rows may be strided), B and C [tokens, N] at columns b_at and c_at of `bc`; a_log
    [channels, N], skip and dt_bias [channels] in the storage type; state [slots, channels, N] 32-bit.  Returns
    (sum_n S C + skip x) * silu(z) rounded to the storage type."""
    _on_gpu(x, dt_pre, bc, z, a_log, skip, dt_bias, state)
    tokens, channels = x.shape
    N = a_log.shape[1]
    for t in (x, dt_pre, bc, z):
        assert t.dtype == torch.float32 and t.stride(1) == 1 and t.shape[0] == tokens
    assert a_log.is_contiguous() and a_log.shape[0] == channels and skip.numel() == channels and dt_bias.numel() == channels
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (channels, N)
    if N > SELECTIVE_SCAN_MAX_STATE:
        raise KernelError(f"selective_scan: a state of {N} entries a channel exceeds {SELECTIVE_SCAN_MAX_STATE}")
    out = torch.empty((tokens, channels), dtype=a_log.dtype, device=x.device)
    _check(lib("selective_scan").lab_selective_scan(
        _ptr(out), out.stride(0), _ptr(x), x.stride(0), _ptr(dt_pre), dt_pre.stride(0), _ptr(bc), bc.stride(0), b_at,
        c_at, _ptr(z), z.stride(0), _ptr(a_log), _ptr(skip), _ptr(dt_bias), _ptr(state), _ptr(ctx.q_start),
        _ptr(ctx.state_slot), ctx.n_requests, channels, N, state.shape[0], int(write), dtype_code(a_log.dtype),
        _stream()), "selective_scan")
    return out


# ----------------------------------------------------------------------------------------
# Routed feed-forward layers (csrc/kernels/moe.cu and the grouped products).
# ----------------------------------------------------------------------------------------
def moe_route(logits: torch.Tensor, experts: int, top: int, gate_col: int = -1, renorm: bool = True):
    """From 32-bit router logits [tokens, >= experts] (column `gate_col` >= 0: the logit of a shared expert's
    gate): (chosen experts [tokens, top] int32, their weights [tokens, top], sigmoid of the gate's logit
    [tokens] or None).  The weights are the chosen scores over their sum, or (`renorm` False) as they are."""
    _on_gpu(logits)
    tokens = logits.shape[0]
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.shape[1] >= experts
    chosen = torch.empty((tokens, top), dtype=torch.int32, device=logits.device)
    weight = torch.empty((tokens, top), dtype=torch.float32, device=logits.device)
    gate = torch.empty((tokens,), dtype=torch.float32, device=logits.device) if gate_col >= 0 else None
    _check(lib("moe").lab_moe_route(_ptr(chosen), _ptr(weight), _ptr(gate), _ptr(logits), logits.stride(0), tokens,
                                    experts, top, gate_col, int(bool(renorm)), _stream()), "moe_route")
    return chosen, weight, gate


def grouped_rows(pairs: int, experts: int, tile: int) -> int:
    """Rows of the layout in which every expert's pairs start on a border of `tile` rows, whatever the choice."""
    return -(-(pairs + experts * (tile - 1)) // tile) * tile


def moe_align(chosen: torch.Tensor, experts: int, tile: int):
    """The (token, choice) pairs laid out in rows grouped by expert: (row_src [rows] int32: the pair at each row
    or -1, tile_group [rows / tile] int32: the expert of each tile or -1, pos_of [pairs] int32: each pair's row)."""
    _on_gpu(chosen)
    pairs = chosen.numel()
    rows = grouped_rows(pairs, experts, tile)
    row_src = torch.empty((rows,), dtype=torch.int32, device=chosen.device)
    tile_group = torch.empty((rows // tile,), dtype=torch.int32, device=chosen.device)
    pos_of = torch.empty((pairs,), dtype=torch.int32, device=chosen.device)
    _check(lib("moe").lab_moe_align(_ptr(row_src), _ptr(tile_group), _ptr(pos_of), _ptr(chosen), pairs, experts, tile,
                                    rows, _stream()), "moe_align")
    return row_src, tile_group, pos_of


def moe_combine(y: torch.Tensor, pos_of: torch.Tensor, weight: torch.Tensor, shared: torch.Tensor | None,
                shared_gate: torch.Tensor | None) -> torch.Tensor:
    """out[t] = sum_k weight[t, k] * y[pos_of[t, k]] (+ shared_gate[t] * shared[t]), 32-bit."""
    _on_gpu(y, pos_of, weight, shared, shared_gate)
    tokens, top = weight.shape
    width = y.shape[1]
    assert y.dtype == torch.float32 and y.is_contiguous() and weight.dtype == torch.float32
    assert shared is None or (shared.dtype == torch.float32 and shared.is_contiguous() and shared.shape == (tokens, width))
    out = torch.empty((tokens, width), dtype=torch.float32, device=y.device)
    _check(lib("moe").lab_moe_combine(_ptr(out), _ptr(y), _ptr(pos_of), _ptr(weight), _ptr(shared), _ptr(shared_gate),
                                      tokens, top, width, _stream()), "moe_combine")
    return out


GROUPED_KERNEL = "auto"     # "auto", "tc" (tcgen05, rows gathered first), "plain" (ordinary units) or "tiles" (their tiled kernel only)
# The experts' products of a step, measured with 8 experts of the 0.5B sizes: the few-rows kernel grows with the
# pairs (62 us at 16, 111 us at 64, 298 us at 254), the tensor cores stay near 60 to 70 us from 16 pairs to 512
# (a tile of 128 rows costs the same part empty), the tiled kernel on the ordinary units near 370 us.
GROUPED_FEW_MAX_PAIRS = 24        # up to this many pairs the few-rows kernel is ahead of the tensor cores
GROUPED_FEW_MAX_PAIRS_PLAIN = 256  # and up to this many ahead of the tiled kernel, where the tensor cores cannot serve


class MoeLayout:
    """The (token, choice) pairs of a step in rows grouped by expert: `row_src` [rows] the pair at each row or -1,
    `tile_group` [rows / tile] the expert of each tile of `tile` rows or -1, `pos_of` [pairs] each pair's row;
    `tc`: the products run on the tensor cores (tiles of their 128 rows); `few`: on the ordinary units by the
    kernel for a handful of rows."""
    __slots__ = ("row_src", "tile_group", "pos_of", "rows", "tile", "tc", "few", "experts")

    def __init__(self, row_src, tile_group, pos_of, tile, tc, few, experts):
        self.row_src, self.tile_group, self.pos_of = row_src, tile_group, pos_of
        self.rows, self.tile, self.tc, self.few, self.experts = row_src.numel(), tile, tc, few, experts


def moe_layout(chosen: torch.Tensor, experts: int, dtype: torch.dtype, width: int, expert_ff: int) -> MoeLayout:
    """Lays a step's pairs out for the experts' products: a handful of pairs (a small decode step) for the few-rows
    kernel on the ordinary units; more on the tensor cores, for bfloat16 and sizes whose rows are whole 16-byte
    units; else on the ordinary units, few-rows up to a few hundred pairs and tiled beyond."""
    pairs = chosen.numel()
    can_tc = (GROUPED_KERNEL not in ("plain", "tiles") and dtype == torch.bfloat16 and not _force_plain and width % 8 == 0
              and expert_ff % 8 == 0)
    tc = can_tc and (GROUPED_KERNEL == "tc" or pairs > GROUPED_FEW_MAX_PAIRS)
    few = (not tc and GROUPED_KERNEL != "tiles"
           and pairs <= (GROUPED_FEW_MAX_PAIRS if can_tc else GROUPED_FEW_MAX_PAIRS_PLAIN))
    tile = int(lib("gemm_tc").lab_gemm_tc_group_rows()) if tc else grouped_tile_rows()
    return MoeLayout(*moe_align(chosen, experts, tile), tile, tc, few, experts)


def moe_gather(x: torch.Tensor, row_src: torch.Tensor, top: int) -> torch.Tensor:
    """out[r] = x[row_src[r] // top]; zeros where row_src is -1."""
    _on_gpu(x, row_src)
    assert x.stride(1) == 1
    out = torch.empty((row_src.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    _check(lib("moe").lab_moe_gather(_ptr(out), _ptr(x), _ptr(row_src), row_src.numel(), top, x.shape[1], x.stride(0),
                                     dtype_code(x.dtype), _stream()), "moe_gather")
    return out


def linear_grouped_tc(x: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, gated: bool = False,
                      out_f32: bool = False, bn: int | None = None, gate_limit: float = 0.0) -> torch.Tensor:
    """Row r of the result is x[r] times the matrix w[tile_group[r // 128]] transposed, on the tcgen05 tensor cores;
    x [rows, K] bfloat16 with rows a multiple of 128, w as for `linear_grouped`.  Rows of tiles whose group is -1
    are left unwritten."""
    _on_gpu(x, w, tile_group)
    rows, K = x.shape
    N = w.shape[1] // 2 if gated else w.shape[1]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not _tc_operands(x, w[0]) or w.shape[2] != K:
        raise KernelError("linear_grouped_tc takes bfloat16 operands with rows of whole 16-byte units")
    assert w.is_contiguous() and w.dim() == 3 and tile_group.numel() * 128 == rows
    out = torch.empty((rows, N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    if bn is None:
        bn = 256 if gated else 128
    _check(lib("gemm_tc").lab_gemm_tc_grouped(_ptr(out), _ptr(x), _ptr(w), rows, N, K, x.stride(0), out.stride(0),
                                              int(gated), int(out_f32), bn, w.shape[0], _ptr(tile_group),
                                              ctypes.c_float(gate_limit), _stream()),
           "gemm_tc_grouped")
    return out


def moe_experts_up(x: torch.Tensor, w_gate_up: torch.Tensor, lay: MoeLayout, top: int, limit: float = 0.0) -> torch.Tensor:
    """silu(W_gate h) * (W_up h) of every pair's token with its expert's matrices, [rows, expert_ff] in the layout
    (`limit` > 0: the capped form of the gate, see `linear_gated`)."""
    if lay.tc:
        return linear_grouped_tc(moe_gather(x, lay.row_src, top), w_gate_up, lay.tile_group, gated=True, gate_limit=limit)
    if lay.few:
        return linear_grouped_few(x, w_gate_up, lay.row_src, top, True, lay.tile_group, lay.tile, gated=True,
                                  gate_limit=limit)
    return linear_grouped(x, w_gate_up, lay.row_src, top, lay.tile_group, lay.rows, gated=True, gate_limit=limit)


def moe_experts_down(act: torch.Tensor, w_down: torch.Tensor, lay: MoeLayout) -> torch.Tensor:
    """W_down of every row's expert on `act` [rows, expert_ff], 32-bit [rows, width]."""
    if lay.tc:
        return linear_grouped_tc(act, w_down, lay.tile_group, out_f32=True)
    if lay.few:
        return linear_grouped_few(act, w_down, lay.row_src, 1, False, lay.tile_group, lay.tile, out_f32=True)
    return linear_grouped(act, w_down, None, 1, lay.tile_group, lay.rows, out_f32=True)


def linear_grouped_few(x: torch.Tensor, w: torch.Tensor, row_src: torch.Tensor, row_div: int, gather: bool,
                       tile_group: torch.Tensor, tile: int, gated: bool = False, out_f32: bool = False,
                       gate_limit: float = 0.0) -> torch.Tensor:
    """`linear_grouped` for a handful of rows: only rows whose `row_src` is not -1 are formed (the others stay
    unwritten); `gather`: row r reads x[row_src[r] // row_div], else x[r]."""
    _on_gpu(x, w, row_src, tile_group)
    rows, K = row_src.numel(), x.shape[1]
    N = w.shape[1] // 2 if gated else w.shape[1]
    assert w.is_contiguous() and w.dim() == 3 and w.shape[2] == K and w.dtype == x.dtype and x.stride(1) == 1
    assert gather or x.shape[0] >= rows
    odt = torch.float32 if (out_f32 or x.dtype == torch.float32) else x.dtype
    out = torch.empty((rows, N), dtype=odt, device=x.device)
    _check(lib("gemm_plain").lab_gemm_plain_grouped_few(
        _ptr(out), _ptr(x), _ptr(w), rows, N, K, x.stride(0), out.stride(0), int(gated),
        ctypes.c_longlong(w.shape[1] * K), _ptr(row_src), int(row_div), int(gather), _ptr(tile_group), int(tile),
        dtype_code(x.dtype), int(out_f32), ctypes.c_float(gate_limit), _stream()), "gemm_plain_grouped_few")
    return out


def grouped_tile_rows() -> int:
    """Rows of a tile of the grouped product on the ordinary units."""
    return int(lib("gemm_plain").lab_gemm_plain_group_rows())


def linear_grouped(x: torch.Tensor, w: torch.Tensor, row_src: torch.Tensor | None, row_div: int,
                   tile_group: torch.Tensor, rows: int, gated: bool = False, out_f32: bool = False,
                   gate_limit: float = 0.0) -> torch.Tensor:
    """Row r of the result is x[row_src[r] // row_div] (row_src None: x[r]) times the matrix w[tile_group[r // tile]]
    transposed; w [groups, out, in], with `gated` [groups, 2 * out, in] (gate rows, then up rows) and the result
    silu(gate) * up.  Rows of tiles whose group is -1 are left unwritten; rows whose source is -1 read zeros."""
    _on_gpu(x, w, row_src, tile_group)
    K = x.shape[1]
    N = w.shape[1] // 2 if gated else w.shape[1]
    assert w.is_contiguous() and w.dim() == 3 and w.shape[2] == K and w.dtype == x.dtype and x.stride(1) == 1
    assert row_src is not None or x.shape[0] >= rows
    odt = torch.float32 if (out_f32 or x.dtype == torch.float32) else x.dtype
    out = torch.empty((rows, N), dtype=odt, device=x.device)
    _check(lib("gemm_plain").lab_gemm_plain_grouped(
        _ptr(out), _ptr(x), _ptr(w), rows, N, K, x.stride(0), out.stride(0), int(gated),
        ctypes.c_longlong(w.shape[1] * K), _ptr(row_src), int(row_div), _ptr(tile_group), dtype_code(x.dtype),
        int(out_f32), ctypes.c_float(gate_limit), _stream()), "gemm_plain_grouped")
    return out


def head_prep_store(proj: torch.Tensor, bias, positions: torch.Tensor, inv_freq: torch.Tensor | None, rot_dims: int, slots,
                    cache_k, cache_v, n_q: int, n_kv: int, dim: int, vdim: int, head: int, k_at: int, v_at: int,
                    dtype: torch.dtype, norm_eps: float = 0.0, q_norm_w=None, k_norm_w=None, q_head_scale=None,
                    temp_coef: float = 0.0, temp_every: int = 0) -> torch.Tensor:
    """`rope_pairs_store` with a norm per head and temperatures on q: after the rotation (`rot_dims` 0: none) every q
    and k head is divided by its root mean square over `dim` (`norm_eps` > 0; eps inside the root) and multiplied by
    a weight of `dim` entries shared by the heads (`q_norm_w`, `k_norm_w`; None: no weight); q is then multiplied by
    `q_head_scale` [n_q] (32-bit; None: 1) and, with `temp_every` > 0, by 1 + temp_coef * ln(floor((pos + 1) /
    temp_every) + 1).  Everything in 32-bit; one rounding where q, k and v leave."""
    _on_gpu(proj, bias, positions, inv_freq, slots, cache_k, cache_v, q_norm_w, k_norm_w, q_head_scale)
    splits = proj.shape[0] if proj.dim() == 3 else 1
    tokens, ld = proj.shape[-2], proj.stride(-2)       # a column slice of a wider product will do
    assert proj.dtype == torch.float32 and proj.stride(-1) == 1 and (proj.dim() == 2 or proj.is_contiguous())
    assert rot_dims == 0 or (inv_freq.dtype == torch.float32 and inv_freq.numel() >= rot_dims // 2)
    assert bias is None or bias.dtype == dtype
    for w in (q_norm_w, k_norm_w):
        assert w is None or (w.dtype == dtype and w.numel() == dim)
    assert q_head_scale is None or (q_head_scale.dtype == torch.float32 and q_head_scale.numel() == n_q)
    write = slots is not None
    n_slots = page_size = 0
    if write:
        assert cache_k.shape == cache_v.shape and cache_k.shape[1] == n_kv and cache_k.shape[3] == head
        assert cache_k.dtype == dtype and cache_k.is_contiguous() and cache_v.is_contiguous()
        page_size = cache_k.shape[2]
        n_slots = cache_k.shape[0] * page_size
    q = torch.empty((tokens, n_q * head), dtype=dtype, device=proj.device)
    _check(lib("rope_pairs").lab_head_prep_store(
        _ptr(q), _ptr(cache_k if write else None), _ptr(cache_v if write else None), _ptr(proj), splits,
        ctypes.c_longlong(tokens * ld), ld, k_at, v_at, _ptr(bias), _ptr(positions), _ptr(inv_freq), rot_dims,
        _ptr(slots), ctypes.c_longlong(n_slots), tokens, n_q, n_kv, dim, vdim, head, max(page_size, 1),
        ctypes.c_float(norm_eps), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(q_head_scale), ctypes.c_float(temp_coef),
        int(temp_every), dtype_code(dtype), _stream()), "head_prep_store")
    return q


# ----------------------------------------------------------------------------------------
# A residual of several streams (csrc/kernels/hyper_stream.cu).
# ----------------------------------------------------------------------------------------
def hyper_max_streams() -> int:
    return int(lib("hyper_stream").lab_hyper_max_streams())


def hyper_expand(x: torch.Tensor, streams: int) -> torch.Tensor:
    """X [tokens, streams, hidden] with every stream a copy of the 32-bit rows x [tokens, hidden]."""
    _on_gpu(x)
    assert x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2
    out = torch.empty((x.shape[0], streams, x.shape[1]), dtype=torch.float32, device=x.device)
    _check(lib("hyper_stream").lab_hyper_expand(_ptr(out), _ptr(x), x.shape[0], streams, x.shape[1], _stream()),
           "hyper_expand")
    return out


def hyper_read_norm(X: torch.Tensor, c_in: torch.Tensor | None, weight: torch.Tensor, eps: float,
                    rows: torch.Tensor | None = None) -> torch.Tensor:
    """u = sum_s c_in[s] X[:, s] (`c_in` None: the plain sum), then u / rms(u) * weight, rounded to the weight's
    storage type; `weight` one number for all coordinates or one per coordinate; `rows`: only those rows."""
    _on_gpu(X, c_in, weight, rows)
    tokens, S, hidden = X.shape
    assert X.dtype == torch.float32 and X.is_contiguous()
    assert c_in is None or (c_in.dtype == torch.float32 and c_in.numel() == S)
    assert weight.numel() in (1, hidden)
    n_out = tokens if rows is None else rows.numel()
    out = torch.empty((n_out, hidden), dtype=weight.dtype, device=X.device)
    _check(lib("hyper_stream").lab_hyper_read_norm(
        _ptr(out), _ptr(X), _ptr(c_in), _ptr(weight), int(weight.numel() == 1 and hidden != 1), _ptr(rows), n_out,
        tokens, S, hidden, ctypes.c_float(eps), dtype_code(weight.dtype), _stream()), "hyper_read_norm")
    return out


def hyper_write(X: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, c_out: torch.Tensor,
                c_in_next: torch.Tensor | None = None, weight_next: torch.Tensor | None = None, eps: float = 0.0):
    """X[:, r] <- sum_s mix[s, r] X[:, s] + c_out[r] * y in place, all streams from the old ones; y a 32-bit result
    [tokens, hidden] or split-K partial products [splits, tokens, hidden] summed in order.  With `c_in_next` and
    `weight_next` it also returns the next sublayer's input, sum_r c_in_next[r] X[:, r] over its root mean square
    times the weight, in the same pass (else None)."""
    _on_gpu(X, y, mix, c_out, c_in_next, weight_next)
    tokens, S, hidden = X.shape
    assert X.dtype == torch.float32 and X.is_contiguous() and y.dtype == torch.float32 and y.is_contiguous()
    assert y.shape[-2:] == (tokens, hidden)
    assert mix.dtype == torch.float32 and mix.numel() == S * S and mix.is_contiguous()
    assert c_out.dtype == torch.float32 and c_out.numel() == S
    splits = y.shape[0] if y.dim() == 3 else 1
    out = None
    if weight_next is not None:
        assert c_in_next.dtype == torch.float32 and c_in_next.numel() == S and weight_next.numel() in (1, hidden)
        out = torch.empty((tokens, hidden), dtype=weight_next.dtype, device=X.device)
    code = dtype_code(weight_next.dtype) if weight_next is not None else F32
    _check(lib("hyper_stream").lab_hyper_write(
        _ptr(X), _ptr(out), _ptr(y), splits, _ptr(mix), _ptr(c_out), _ptr(c_in_next if out is not None else None),
        _ptr(weight_next), int(weight_next is not None and weight_next.numel() == 1 and hidden != 1), tokens, S, hidden,
        ctypes.c_float(eps), code, _stream()), "hyper_write")
    return out


def normed_sum(a: torch.Tensor, wa: torch.Tensor, ca: float, b: torch.Tensor | None, wb: torch.Tensor | None, cb: float,
               eps: float) -> torch.Tensor:
    """ca * a / rms(a) * wa + cb * b / rms(b) * wb in 32-bit: a and b 32-bit products [tokens, hidden] or split-K
    partial products (summed in order), each normed over the hidden size with its own weight; b may be None."""
    _on_gpu(a, wa, b, wb)
    tokens, hidden = a.shape[-2:]
    assert a.dtype == torch.float32 and a.is_contiguous() and wa.numel() == hidden
    if b is not None:
        assert b.dtype == torch.float32 and b.is_contiguous() and b.shape[-2:] == (tokens, hidden)
        assert wb.numel() == hidden and wb.dtype == wa.dtype
    out = torch.empty((tokens, hidden), dtype=torch.float32, device=a.device)
    _check(lib("hyper_stream").lab_normed_sum(
        _ptr(out), _ptr(a), a.shape[0] if a.dim() == 3 else 1, _ptr(wa), ctypes.c_float(ca), _ptr(b),
        (b.shape[0] if b.dim() == 3 else 1) if b is not None else 0, _ptr(wb), ctypes.c_float(cb), tokens, hidden,
        ctypes.c_float(eps), dtype_code(wa.dtype), _stream()), "normed_sum")
    return out


def scale_rows(x: torch.Tensor, c: float) -> torch.Tensor:
    """x <- x * c in place (32-bit)."""
    _on_gpu(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(lib("hyper_stream").lab_scale_rows(_ptr(x), ctypes.c_longlong(x.numel()), ctypes.c_float(c), _stream()),
           "scale_rows")
    return x


# ----------------------------------------------------------------------------------------
# A matrix memory with exponential gates (csrc/kernels/matrix_memory.cu) around `decay_scan`.
# ----------------------------------------------------------------------------------------
def memory_value_width(vdim: int) -> int:
    """Columns a head's values take in the recurrence: vdim, one column of ones for the normaliser, and zeros up
    to a multiple of four (16-byte rows)."""
    return (vdim + 1 + 3) // 4 * 4


def memory_gates(proj: torch.Tensor, v_at: int, i_at: int, f_at: int, b_i: torch.Tensor, b_f: torch.Tensor, heads: int,
                 vdim: int, cap: float):
    """From the 32-bit input projection: gates [tokens, 2, heads] (i = cap tanh((z_i + b_i) / cap), f =
    logsigmoid(cap tanh((z_f + b_f) / cap))) and the values [tokens, heads * memory_value_width(vdim)] with their
    column of ones."""
    _on_gpu(proj, b_i, b_f)
    tokens = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and b_i.numel() == heads and b_f.numel() == heads
    assert b_i.dtype == b_f.dtype
    vpad = memory_value_width(vdim)
    gates = torch.empty((tokens, 2, heads), dtype=torch.float32, device=proj.device)
    values = torch.empty((tokens, heads * vpad), dtype=torch.float32, device=proj.device)
    _check(lib("matrix_memory").lab_memory_gates(
        _ptr(gates), _ptr(values), _ptr(proj), proj.stride(0), v_at, i_at, f_at, _ptr(b_i), _ptr(b_f), tokens, heads,
        vdim, vpad, ctypes.c_float(cap), dtype_code(b_i.dtype), _stream()), "memory_gates")
    return gates, values


def memory_stabilize(gates: torch.Tensor, m_state: torch.Tensor, ctx, write: bool = True) -> torch.Tensor:
    """Walks every request's rows in order: m <- max(f + m, i) from the request's slot of `m_state` [slots, heads];
    `gates` [tokens, 2, heads] become the state's decay exp(f + m_before - m) and the key's scale exp(i - m) of each
    row; returns m of every row [tokens, heads].  With `write` the last m goes back to the slot."""
    _on_gpu(gates, m_state)
    tokens, _, heads = gates.shape
    assert gates.dtype == torch.float32 and gates.is_contiguous()
    assert m_state.dtype == torch.float32 and m_state.is_contiguous() and m_state.shape[1:] == (heads,)
    m = torch.empty((tokens, heads), dtype=torch.float32, device=gates.device)
    _check(lib("matrix_memory").lab_memory_stabilize(
        _ptr(gates), _ptr(m), _ptr(m_state), _ptr(ctx.q_start), _ptr(ctx.state_slot), ctx.n_requests, m_state.shape[0],
        heads, int(write), _stream()), "memory_stabilize")
    return m


def memory_finish(o: torch.Tensor, m: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, ctx, heads: int, vdim: int,
                  q_scale: float, floor: float, eps: float, mult: float = 1.0, out: torch.Tensor | None = None):
    """From the recurrence's output o [tokens, heads * memory_value_width(vdim)] (S^T q and, in column vdim, n . q,
    both for the unscaled q): y = q_scale S^T q / (max(|q_scale n . q|, exp(-m)) + floor); every head over its root
    mean square; times `weight` [heads * vdim], times sigmoid(gate) (32-bit column slice), times `mult`; rounded
    to the weight's storage type.  Rows of requests without a state slot (padding) leave as zeros."""
    _on_gpu(o, m, gate, weight, out)
    tokens = o.shape[0]
    vpad = memory_value_width(vdim)
    assert o.dtype == torch.float32 and o.is_contiguous() and o.shape[1] == heads * vpad
    assert m.dtype == torch.float32 and m.is_contiguous() and m.shape == (tokens, heads)
    assert gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape == (tokens, heads * vdim)
    assert weight.numel() == heads * vdim
    if out is None:
        out = torch.empty((tokens, heads * vdim), dtype=weight.dtype, device=o.device)
    assert out.dtype == weight.dtype and out.stride(1) == 1 and out.shape == (tokens, heads * vdim)
    _check(lib("matrix_memory").lab_memory_finish(
        _ptr(out), out.stride(0), _ptr(o), _ptr(m), _ptr(gate), gate.stride(0), _ptr(weight), tokens, heads, vdim, vpad,
        ctypes.c_float(q_scale), ctypes.c_float(floor), ctypes.c_float(eps), ctypes.c_float(mult),
        _ptr(ctx.row_req), _ptr(ctx.state_slot), dtype_code(weight.dtype), _stream()), "memory_finish")
    return out
