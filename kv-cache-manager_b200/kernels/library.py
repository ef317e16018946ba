"""Python face of ``libkvcm_cuda.so``: one function per exported launcher.

Every function checks what the kernel assumes (device, dtype, contiguity, shapes), passes raw
pointers and the current torch CUDA stream, and raises ``KernelError`` on a non-zero return.
There is no fallback of any kind: without the compiled library, or with tensors that are not
on a CUDA device, these functions raise.  ``launch_count()`` counts launches of this library's
kernels (used by the benchmark's ``gpu_launches``).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc.build import load_cuda

_SUFFIX = {torch.float32: "f32", torch.bfloat16: "bf16"}
_ERR_UNSUPPORTED = 10001
_launches = 0


class KernelError(RuntimeError):
    pass


def launch_count() -> int:
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def add_launches(n: int) -> None:
    """Launches made by the C++ request loop, which calls the launchers without passing here."""
    global _launches
    _launches += int(n)


def profiling() -> bool:
    return _profile is not None


class DeviceBackend(ctypes.Structure):
    """Opaque room for the table of device functions that the kernel library fills for the C++
    request loop (csrc/include/device_backend.h): 23 function pointers."""
    _fields_ = [("slots", ctypes.c_void_p * 23)]


_backend = None


def device_backend_address() -> int:
    """Address of the filled table (kept alive for the life of the process)."""
    global _backend
    if _backend is None:
        b = DeviceBackend()
        size = int(_lib().kvcm_device_backend(ctypes.byref(b)))
        if size != ctypes.sizeof(DeviceBackend):
            raise KernelError("device backend: the table of the library has another layout")
        _backend = b
    return ctypes.addressof(_backend)


def _lib():
    return load_cuda()


def _suffix(t: torch.Tensor) -> str:
    try:
        return _SUFFIX[t.dtype]
    except KeyError:
        raise KernelError(f"kernels exist for float32 and bfloat16 storage, not {t.dtype}") from None


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    # (the raw handle of the current stream, without building a Stream object: a launch of a small
    # kernel costs about 10 us of host time, and a third of it was this)
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel called with a tensor that is not on a CUDA device "
                              "(this engine has no CPU path)")


_profile = None          # while profiling: [(kernel family, event recorded after its launch)]


def profile_start() -> None:
    """Starts per-family timing: from now on an event is recorded after every launch of this
    library's kernels (and after library products, which call ``profile_mark``).  The stream runs
    in order, so the time between two consecutive events is the time of the later launch (its
    launch gap included).  For eager steps only: events cannot be recorded into a CUDA graph."""
    global _profile
    first = torch.cuda.Event(enable_timing=True)
    first.record()
    _profile = [("", first)]


def profile_mark(name: str) -> None:
    if _profile is not None:
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        _profile.append((name, e))


def profile_stop() -> dict:
    """Ends profiling; {family: (launches, device milliseconds)}."""
    global _profile
    marks, _profile = _profile or [], None
    torch.cuda.synchronize()
    out: dict = {}
    for (_, before), (name, after) in zip(marks, marks[1:]):
        calls, ms = out.get(name, (0, 0.0))
        out[name] = (calls + 1, ms + before.elapsed_time(after))
    return out


def _check(rc: int, name: str, detail: str = "") -> None:
    global _launches
    _launches += 1
    if _profile is not None:
        profile_mark(name)
    if rc == 0:
        return
    if rc == _ERR_UNSUPPORTED:
        raise KernelError(f"{name}: sizes not supported by this kernel {detail}")
    raise KernelError(f"{name}: CUDA error {rc} at launch {detail}")


_I32 = torch.int32


def embed(ids: torch.Tensor, table: torch.Tensor, x: torch.Tensor) -> None:
    """x[t,:] = float(table[ids[t],:]); x is float32 [T, H]."""
    _cuda(ids, table, x)
    T, H = x.shape
    _need(ids.dtype == _I32 and ids.numel() >= T, "embed: ids must be int32 [T]")
    _need(x.dtype == torch.float32 and x.is_contiguous() and table.is_contiguous(), "embed: layout")
    _need(table.shape[1] == H, "embed: table width != hidden")
    fn = getattr(_lib(), "kvcm_embed_" + _suffix(table))
    _check(fn(_p(ids), _p(table), _p(x), T, H, table.shape[0], _stream()), "embed")


def rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
            out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """Optional x += delta, then out = weight * round(x * rsqrt(mean(x^2)+eps)).

    x float32 [T,H] (updated in place unless ``rows`` gathers); delta/out in the storage dtype;
    weight in the storage dtype or float32."""
    _cuda(x, delta, weight, out, rows)
    H = x.shape[1]
    n = out.shape[0]
    _need(x.dtype == torch.float32 and x.is_contiguous(), "rmsnorm: x must be contiguous float32")
    _need(out.is_contiguous() and out.shape[1] == H and weight.numel() == H, "rmsnorm: shapes")
    _need(delta is None or (delta.dtype == out.dtype and delta.is_contiguous()
                            and delta.shape == x.shape), "rmsnorm: delta must match x in shape")
    _need(weight.dtype in (torch.float32, out.dtype), "rmsnorm: weight dtype")
    if rows is None:
        _need(n == x.shape[0], "rmsnorm: out rows != x rows")
    else:
        _need(rows.dtype == _I32 and rows.numel() >= n, "rmsnorm: rows must be int32 [n]")
    fn = getattr(_lib(), "kvcm_rmsnorm_" + _suffix(out))
    wf32 = int(weight.dtype == torch.float32)
    _check(fn(_p(x), _p(delta), _p(weight), wf32, _p(out), _p(rows), n, H,
              ctypes.c_float(eps), _stream()), "rmsnorm", f"(hidden={H})")


def add_residual(x: torch.Tensor, delta: torch.Tensor) -> None:
    _cuda(x, delta)
    _need(x.dtype == torch.float32 and x.is_contiguous() and delta.is_contiguous()
          and x.shape == delta.shape, "add_residual: shapes")
    fn = getattr(_lib(), "kvcm_add_residual_" + _suffix(delta))
    _check(fn(_p(x), _p(delta), ctypes.c_longlong(x.numel()), _stream()), "add_residual")


def rope_cache(qkv: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
               rotary_dim: int, interleaved: bool, slot_mapping: Optional[torch.Tensor],
               k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
               nh: int, nkv: int, hd: int, block_size: int, write_cache: bool = True) -> None:
    """Rotary encoding of the q and k heads of the fused rows in place, then K and V of each row
    are written to its page slot.  k_cache/v_cache: one layer, [pages, nkv, block, hd]."""
    _cuda(qkv, positions, inv_freq, slot_mapping, k_cache, v_cache)
    T = qkv.shape[0]
    _need(qkv.stride(1) == 1 and qkv.shape[1] >= (nh + 2 * nkv) * hd, "rope_cache: qkv row too short")
    _need(positions.dtype == _I32 and positions.numel() >= T, "rope_cache: positions int32 [T]")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 >= rotary_dim,
              "rope_cache: inv_freq must be float32 [rotary_dim/2]")
    if write_cache:
        _need(slot_mapping is not None and slot_mapping.dtype == _I32 and slot_mapping.numel() >= T,
              "rope_cache: slot_mapping int32 [T]")
        _need(k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype and k_cache.is_contiguous()
              and v_cache.is_contiguous(), "rope_cache: cache dtype/layout")
        _need(tuple(k_cache.shape[1:]) == (nkv, block_size, hd), "rope_cache: cache page shape")
    fn = getattr(_lib(), "kvcm_rope_cache_" + _suffix(qkv))
    _check(fn(_p(qkv), qkv.stride(0), _p(positions), _p(inv_freq), rotary_dim, int(interleaved),
              _p(slot_mapping), _p(k_cache), _p(v_cache), T, nh, nkv, hd, block_size,
              int(write_cache), _stream()), "rope_cache", f"(rotary_dim={rotary_dim}, hd={hd})")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, table: torch.Tensor) -> None:
    """table[t] = [cos(positions[t] * inv_freq) | sin(...)] (float32 [T, 2 * len(inv_freq)]): the
    angles of a step, which are the same in every layer."""
    _cuda(positions, inv_freq, table)
    T, width = table.shape
    _need(positions.dtype == _I32 and positions.numel() >= T, "rope_table: positions int32 [T]")
    _need(inv_freq.dtype == torch.float32 and table.dtype == torch.float32 and table.is_contiguous()
          and width == 2 * inv_freq.numel(), "rope_table: float32 inv_freq [hd/2] and table [T, hd]")
    _check(_lib().kvcm_rope_table_f32(_p(positions), _p(inv_freq), T, width // 2, _p(table), _stream()), "rope_table")


def rope_cache_table(qkv: torch.Tensor, table: torch.Tensor, slot_mapping: Optional[torch.Tensor],
                     k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], nh: int, nkv: int, hd: int,
                     block_size: int, write_cache: bool = True) -> None:
    """``rope_cache`` for bfloat16 rows rotated over the whole head in rotate-half pairs, with the
    cosines and sines read from ``table`` (``rope_table``): the same bits."""
    _cuda(qkv, table, slot_mapping, k_cache, v_cache)
    T = qkv.shape[0]
    _need(qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and qkv.shape[1] >= (nh + 2 * nkv) * hd,
          "rope_cache_table: bfloat16 rows of q, k and v heads")
    _need(table.dtype == torch.float32 and table.is_contiguous() and tuple(table.shape) == (T, hd),
          "rope_cache_table: table float32 [T, hd]")
    if write_cache:
        _need(slot_mapping is not None and slot_mapping.dtype == _I32 and slot_mapping.numel() >= T,
              "rope_cache_table: slot_mapping int32 [T]")
        _need(k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype and k_cache.is_contiguous()
              and v_cache.is_contiguous() and tuple(k_cache.shape[1:]) == (nkv, block_size, hd),
              "rope_cache_table: cache dtype/layout")
    rc = _lib().kvcm_rope_cache_table_bf16(_p(qkv), qkv.stride(0), _p(table), _p(slot_mapping), _p(k_cache), _p(v_cache),
                                           T, nh, nkv, hd, block_size, int(write_cache), _stream())
    _check(rc, "rope_cache_table", f"(hd={hd}, row stride {qkv.stride(0)})")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(gate_up, out)
    T, I = out.shape
    _need(gate_up.is_contiguous() and out.is_contiguous() and gate_up.shape == (T, 2 * I)
          and gate_up.dtype == out.dtype, "silu_mul: gate_up must be [T, 2I]")
    fn = getattr(_lib(), "kvcm_silu_mul_" + _suffix(out))
    _check(fn(_p(gate_up), _p(out), T, I, _stream()), "silu_mul")


def gather_rows(src: torch.Tensor, rows: torch.Tensor, dst: torch.Tensor) -> None:
    _cuda(src, rows, dst)
    n, W = dst.shape
    _need(src.is_contiguous() and dst.is_contiguous() and src.shape[1] == W and src.dtype == dst.dtype
          and rows.dtype == _I32 and rows.numel() >= n, "gather_rows: shapes")
    fn = getattr(_lib(), "kvcm_gather_rows_" + _suffix(dst))
    _check(fn(_p(src), _p(rows), _p(dst), n, W, _stream()), "gather_rows")


def gemm_plain(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> None:
    """y[M,N] = x[M,K] @ w[N,K]^T with float accumulation in a fixed k order (plain kernel)."""
    _cuda(x, w, y)
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and y.shape == (M, N), "gemm_plain: shapes")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and y.stride(1) == 1, "gemm_plain: rows must be dense")
    _need(x.dtype == w.dtype, "gemm_plain: operand dtypes differ")
    if x.dtype == torch.float32:
        _need(y.dtype == torch.float32, "gemm_plain: float32 operands need a float32 result")
        name = "kvcm_gemm_plain_f32"
    elif x.dtype == torch.bfloat16:
        name = "kvcm_gemm_plain_bf16" if y.dtype == torch.bfloat16 else "kvcm_gemm_plain_bf16_f32out"
        _need(y.dtype in (torch.bfloat16, torch.float32), "gemm_plain: result dtype")
    else:
        raise KernelError(f"gemm_plain: dtype {x.dtype}")
    _check(getattr(_lib(), name)(_p(x), _p(w), _p(y), M, N, K, x.stride(0), w.stride(0), y.stride(0),
                                 _stream()), "gemm_plain")


def attention_plain(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_tables: torch.Tensor, row_seq: torch.Tensor, positions: torch.Tensor,
                    nh: int, nkv: int, hd: int, scale: float, window: int = 0, softcap: float = 0.0,
                    sink: Optional[torch.Tensor] = None, keep_first: int = 0) -> None:
    """Row-per-query paged attention.  q: [T, >= nh*hd] (row stride free), out: [T, nh*hd];
    caches [pages, nkv, block, hd]; block_tables int32 [S, max_blocks].  ``softcap`` > 0 caps the
    scaled scores as cap * tanh(score / cap); ``sink`` (float32 [nh]) adds exp(sink) of each head to
    its softmax denominators; with a window, ``keep_first`` > 0 keeps a request's first keys visible to every row."""
    _cuda(q, out, k_cache, v_cache, block_tables, row_seq, positions, sink)
    _need(sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == nh),
          "attention: sink float32 [heads]")
    T = out.shape[0]
    _need(q.stride(1) == 1 and out.stride(1) == 1, "attention: rows must be dense")
    _need(q.dtype == out.dtype == k_cache.dtype == v_cache.dtype, "attention: dtypes differ")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape[1] == nkv
          and k_cache.shape[3] == hd, "attention: cache page shape")
    _need(block_tables.dtype == _I32 and block_tables.is_contiguous() and block_tables.dim() == 2,
          "attention: block_tables int32 [S, max_blocks]")
    _need(row_seq.dtype == _I32 and positions.dtype == _I32 and row_seq.numel() >= T
          and positions.numel() >= T, "attention: row_seq/positions int32 [T]")
    fn = getattr(_lib(), "kvcm_attention_plain_keep_" + _suffix(q))
    _check(fn(_p(q), q.stride(0), _p(out), out.stride(0), _p(k_cache), _p(v_cache), _p(block_tables),
              block_tables.shape[1], _p(row_seq), _p(positions), T, nh, nkv, hd, k_cache.shape[2],
              ctypes.c_float(scale), int(window), ctypes.c_float(softcap), _p(sink), int(keep_first), _stream()), "attention_plain",
           f"(hd={hd}, nh={nh}, nkv={nkv})")


# Kernel families whose bounded waits report through an error word, in the order of the status
# index that the sampling kernels write (csrc/cuda/sampling.cu: status_words).
STATUS_FAMILIES = ("gemm_stream", "gemm_tcgen05", "gemm_tcgen05_pair", "gemm_tcgen05_splitk", "attention_tcgen05",
                   "moe_tcgen05")


def describe_status(first: int, word: int) -> str:
    """Text for a status pair written by the sampling kernels: ``first`` = 1 + index of the kernel
    family whose error word was set (0 = none), ``word`` = (code << 16) | block."""
    name = STATUS_FAMILIES[first - 1] if 1 <= first <= len(STATUS_FAMILIES) else f"family {first}"
    return (f"{name}: a bounded wait ran out on the device (code {(word >> 16) & 0xffff}, block {word & 0xffff}); "
            f"the outputs of this step are not valid")


def raise_on_status(first: int, word: int) -> None:
    """Raises ``KernelError`` when the status pair of a step names a kernel family; clears the
    device's error words first so that the next step starts clean."""
    if not first:
        return
    clear_errors()
    raise KernelError(describe_status(int(first), int(word)))


def clear_errors() -> None:
    """Reads and clears every family's error word (synchronises with the device)."""
    for fn in (stream_error, tcgen05_error, pair_error, splitk_error, attention_tcgen05_error, moe_tcgen05_error):
        fn()


def check_errors() -> None:
    """Host-side read of every family's error word (synchronises); raises if one is set.  For paths
    that synchronise anyway (scoring, replay); generation reads the status pair beside its tokens."""
    for i, fn in enumerate((stream_error, tcgen05_error, pair_error, splitk_error, attention_tcgen05_error,
                            moe_tcgen05_error)):
        word = fn()
        if word:
            clear_errors()
            raise KernelError(describe_status(i + 1, word))


def _status_ptr(status: Optional[torch.Tensor]):
    if status is None:
        return None
    _cuda(status)
    _need(status.dtype == _I32 and status.numel() >= 2 and status.is_contiguous(), "status: int32 [2]")
    return _p(status)


def argmax(logits: torch.Tensor, out: torch.Tensor, status: Optional[torch.Tensor] = None) -> None:
    """out[r] = first index of the row's maximum.  ``status`` (int32 [2], optional) receives the
    first error word that a kernel of this step has set (see ``describe_status``)."""
    _cuda(logits, out)
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous() and out.dtype == _I32
          and out.numel() >= R, "argmax: logits float32 [R,V], out int32 [R]")
    _check(_lib().kvcm_argmax_status_f32(_p(logits), _p(out), R, V, _status_ptr(status), _stream()), "argmax")


def sample(logits: torch.Tensor, temperature: torch.Tensor, seed: torch.Tensor,
           request_id: torch.Tensor, position: torch.Tensor, out: torch.Tensor,
           status: Optional[torch.Tensor] = None) -> None:
    """Per row: temperature <= 0 -> argmax; else one draw from softmax(logits / temperature) with a
    uniform number that depends only on (seed, request id, position).  ``status`` as in ``argmax``."""
    _cuda(logits, temperature, seed, request_id, position, out)
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "sample: logits float32 [R,V]")
    _need(temperature.dtype == torch.float32 and seed.dtype == torch.int64
          and request_id.dtype == torch.int64 and position.dtype == _I32 and out.dtype == _I32,
          "sample: temperature f32, seed/request_id i64, position/out i32")
    _need(min(temperature.numel(), seed.numel(), request_id.numel(), position.numel(),
              out.numel()) >= R, "sample: per-row arrays shorter than the number of rows")
    _check(_lib().kvcm_sample_status_f32(_p(logits), _p(temperature), _p(seed), _p(request_id),
                                         _p(position), _p(out), R, V, _status_ptr(status), _stream()), "sample")


# ------------------------------------------------------------------ dispatch of attention

def paged_attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_tables: torch.Tensor, ctx, nh: int, nkv: int, hd: int, scale: float,
                    window: int = 0, softcap: float = 0.0, sink: Optional[torch.Tensor] = None,
                    keep_first: int = 0) -> None:
    """Attention of all rows of a step.  Rows [0, ctx.decode_seqs) are single-row entries, the
    rest are the rows of longer portions.  ``ctx.options['attention']``: 'plain' forces the plain
    kernel for every row; float32 storage always uses it (the true 32-bit path)."""
    mode = ctx.options.get("attention", "auto")
    if mode == "plain" or q.dtype == torch.float32 or not fast_attention_supported(nh, nkv, hd, k_cache.shape[2]):
        attention_plain(q, out, k_cache, v_cache, block_tables, ctx.row_seq, ctx.positions,
                        nh, nkv, hd, scale, window, softcap, sink, keep_first)
        return
    nd = ctx.decode_seqs
    if nd > 0:
        attention_decode(q[:nd], out[:nd], k_cache, v_cache, block_tables, ctx, nh, nkv, hd, scale, window, softcap, sink,
                         keep_first)
    if ctx.rows > nd:
        attention_prefill(q, out, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, scale, window, softcap, sink,
                          keep_first)


def fast_attention_supported(nh: int, nkv: int, hd: int, block_size: int) -> bool:
    return nkv > 0 and nh % nkv == 0 and bool(_lib().kvcm_attention_fast_supports(int(hd)))


_SM_COUNT = {}


def sm_count(device) -> int:
    d = torch.device(device)
    if d not in _SM_COUNT:
        _SM_COUNT[d] = torch.cuda.get_device_properties(d).multi_processor_count
    return _SM_COUNT[d]


KEY_TILE = 64
CLUSTER_PARTS = 8           # kvcm_attention_decode_cluster_parts()


_RESIDENT = {}


def _decode_resident_blocks(hd: int, device) -> int:
    key = (int(hd), torch.device(device))
    if key not in _RESIDENT:
        n = int(_lib().kvcm_attention_decode_resident_blocks(int(hd)))
        _RESIDENT[key] = n if n > 0 else 3 * sm_count(device)
    return _RESIDENT[key]


def decode_partitions(seqs: int, nh: int, nkv: int, hd: int, max_ctx: int, device, version: str = "auto",
                      force_parts: int = 0):
    """How the decode kernel splits the context: (keys per partition, number of partitions).

    'v1': the whole context in one block per (request, KV head).  'v2'/'auto': as many partitions
    as keep the whole grid resident at once (a second wave of blocks costs more than longer
    partitions), each at least 128 keys long, and no more than the 8 that merge inside one cluster
    unless that would leave partitions of more than 512 keys.  Measured on a B200 over batches
    1..128 and contexts 512..8192.  (The reference fixes 512 keys per partition,
    src/cuda/paged_attention.cu:22.)  ``force_parts`` > 0 asks for that many partitions (tuning
    and tests)."""
    max_ctx = max(int(max_ctx), 1)
    whole = (max_ctx + KEY_TILE - 1) // KEY_TILE * KEY_TILE
    if version == "v1":
        return whole, 1
    G = nh // nkv
    blocks = max(1, seqs * nkv * ((G + 15) // 16))
    if force_parts > 0:
        parts = min(int(force_parts), max(1, whole // KEY_TILE))
    else:
        parts = max(1, min(_decode_resident_blocks(hd, device) // blocks, max_ctx // 128))
        if parts > CLUSTER_PARTS:
            parts = max(CLUSTER_PARTS, min(parts, (max_ctx + 511) // 512))
    size = ((max_ctx + parts - 1) // parts + KEY_TILE - 1) // KEY_TILE * KEY_TILE
    parts = (max_ctx + size - 1) // size
    return size, parts


def attention_decode(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     block_tables: torch.Tensor, ctx, nh: int, nkv: int, hd: int, scale: float,
                     window: int = 0, softcap: float = 0.0, sink: Optional[torch.Tensor] = None,
                     keep_first: int = 0) -> None:
    """Single-row entries: q/out hold one row per request, in the order of the batch's entries.
    ``softcap`` / ``sink`` as in ``attention_plain``."""
    _cuda(q, out, k_cache, v_cache, block_tables, sink)
    _need(sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == nh),
          "attention_decode: sink float32 [heads]")
    S = q.shape[0]
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16,
          "attention_decode: bfloat16 only")
    _need(q.stride(1) == 1 and out.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous(),
          "attention_decode: layout")
    _need(q.data_ptr() % 16 == 0 and (q.stride(0) * 2) % 16 == 0, "attention_decode: q rows must be 16-byte aligned")
    size, parts = decode_partitions(S, nh, nkv, hd, ctx.max_decode_ctx, q.device,
                                    ctx.options.get("attn_version", "auto"), int(ctx.options.get("attn_parts", 0)))
    scratch = None
    # Up to 8 partitions merge inside a thread-block cluster; more go through scratch memory
    # and a merge kernel ('attn_merge': 'kernel' forces that path).
    in_cluster = 1 < parts <= CLUSTER_PARTS and ctx.options.get("attn_merge", "cluster") == "cluster"
    if parts > 1 and not in_cluster:
        n = S * nh * parts * (hd + 2)          # partial outputs + (max, sum) per partition
        scratch = torch.empty(n, dtype=torch.float32, device=q.device)
    rc = _lib().kvcm_attention_decode_keep_bf16(
        _p(q), q.stride(0), _p(out), out.stride(0), _p(k_cache), _p(v_cache), _p(block_tables),
        block_tables.shape[1], _p(ctx.seq_ctx_len), S, nh, nkv, hd, k_cache.shape[2],
        ctypes.c_float(scale), int(window), int(keep_first), size, parts, _p(scratch), int(in_cluster), ctypes.c_float(softcap), _p(sink),
        _stream())
    _check(rc, "attention_decode", f"(hd={hd}, nh={nh}, nkv={nkv})")
    if parts > 1 and not in_cluster:
        global _launches
        _launches += 1                      # the merge kernel


def attention_prefill(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      block_tables: torch.Tensor, ctx, nh: int, nkv: int, hd: int, scale: float,
                      window: int = 0, softcap: float = 0.0, sink: Optional[torch.Tensor] = None,
                      keep_first: int = 0) -> None:
    """Rows of portions longer than one token; q/out are the step's full row arrays.
    ``ctx.options['attn_prefill']``: 'tcgen05' | 'mma' force a kernel; 'auto' takes the tcgen05
    kernel where it supports the sizes (head_dim 64 or 128, 256 when keys and values are the same pages; pages of
    8 to 64 keys dividing 64, or multiples of 64)."""
    _cuda(q, out, k_cache, v_cache, block_tables, sink)
    _need(sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == nh),
          "attention_prefill: sink float32 [heads]")
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16,
          "attention_prefill: bfloat16 only")
    _need(q.stride(1) == 1 and out.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous(),
          "attention_prefill: layout")
    _need(q.data_ptr() % 16 == 0 and (q.stride(0) * 2) % 16 == 0, "attention_prefill: q rows must be 16-byte aligned")
    _need(ctx.tile_rows == 64, "attention_prefill: the batch must be tiled in 64 query rows")
    mode = ctx.options.get("attn_prefill", "auto")
    B = k_cache.shape[2]
    kept = int(keep_first) if window > 0 else 0
    shared_kv = k_cache.data_ptr() == v_cache.data_ptr()
    if mode != "mma" and (mode == "tcgen05" or prefill_tcgen05_supported(hd, B, shared_kv)):
        _need(out.data_ptr() % 16 == 0 and out.stride(0) % 8 == 0, "attention_prefill: out rows must be 16-byte aligned")
        rc = _lib().kvcm_attention_prefill_tcgen05_bf16(
            _p(q), q.stride(0), q.shape[0], _p(out), out.stride(0), _p(k_cache), _p(v_cache), k_cache.shape[0],
            _p(block_tables), block_tables.shape[1], _p(ctx.tile_seq), _p(ctx.tile_q0), _p(ctx.seq_q_start),
            _p(ctx.seq_q_len), _p(ctx.seq_ctx_len), ctx.prefill_tiles, nh, nkv, hd, B, ctypes.c_float(scale),
            int(window), kept, ctypes.c_float(softcap), _p(sink), _stream())
        _check(rc, "attention_prefill_tcgen05", f"(hd={hd}, nh={nh}, nkv={nkv}, block={B})")
        return
    rc = _lib().kvcm_attention_prefill_keep_bf16(
        _p(q), q.stride(0), _p(out), out.stride(0), _p(k_cache), _p(v_cache), _p(block_tables),
        block_tables.shape[1], _p(ctx.tile_seq), _p(ctx.tile_q0), _p(ctx.seq_q_start), _p(ctx.seq_q_len),
        _p(ctx.seq_ctx_len), ctx.prefill_tiles, nh, nkv, hd, B, ctypes.c_float(scale),
        int(window), kept, ctypes.c_float(softcap), _p(sink), _stream())
    _check(rc, "attention_prefill", f"(hd={hd}, nh={nh}, nkv={nkv})")


def prefill_tcgen05_supported(hd: int, block_size: int, shared_kv: bool = False) -> bool:
    """``shared_kv``: keys and values are the same pages (attention over a cached latent), which opens head_dim 256."""
    return bool(_lib().kvcm_attention_tcgen05_supports_kv(int(hd), int(block_size), int(bool(shared_kv))))


def attention_tcgen05_error() -> int:
    """Error word of the tcgen05 attention kernel: 0, or (code << 16 | block) of a bounded wait that
    ran out.  Reading clears it.  Synchronises the device."""
    return int(_lib().kvcm_attention_tcgen05_error())

def stream_gemm_supported(M: int, N: int, K: int) -> bool:
    """True when the TMA-pipelined weight-streaming kernel takes this product."""
    return bool(_lib().kvcm_gemm_stream_supports(int(M), int(N), int(K)))


def gemm_stream(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> None:
    """y[M,N] = x[M,K] @ w[N,K]^T for M <= 16 with W streamed through a shared-memory ring by bulk
    asynchronous copies (bfloat16 operands, float accumulation, bfloat16 or float result)."""
    _cuda(x, w, y)
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and y.shape == (M, N), "gemm_stream: shapes")
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and y.dtype in (torch.bfloat16, torch.float32),
          "gemm_stream: bfloat16 operands, bfloat16 or float32 result")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and y.stride(1) == 1, "gemm_stream: rows must be dense")
    rc = _lib().kvcm_gemm_stream_bf16(_p(x), _p(w), _p(y), M, N, K, x.stride(0), w.stride(0), y.stride(0),
                                      int(y.dtype == torch.float32), sm_count(x.device), _stream())
    _check(rc, "gemm_stream", f"(M={M}, N={N}, K={K})")


def gemm_stream_relu_sq(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> None:
    """y = max(bfloat16(x @ w^T), 0)^2 in bfloat16: the streaming product of ``gemm_stream`` with the
    activation of an ungated feed-forward in its epilogue (the same roundings as product, then ``relu_sq``)."""
    _cuda(x, w, y)
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and y.shape == (M, N) and x.dtype == w.dtype == y.dtype == torch.bfloat16
          and x.stride(1) == 1 and w.stride(1) == 1 and y.stride(1) == 1, "gemm_stream_relu_sq: bfloat16 [M,K] x [N,K]")
    rc = _lib().kvcm_gemm_stream_relu_sq_bf16(_p(x), _p(w), _p(y), M, N, K, x.stride(0), w.stride(0), y.stride(0),
                                              sm_count(x.device), _stream())
    _check(rc, "gemm_stream", f"(M={M}, N={N}, K={K}, relu_sq)")


def stream_test_hooks(wait_limit_ns: int = 0, skip_stage: int = -1) -> None:
    """For tests of the failure path: the streaming product's wait limit (0 = its default) and a
    stage of every block whose copy is left out (-1 = none), so that a wait runs out."""
    rc = _lib().kvcm_stream_test_hooks(ctypes.c_uint64(int(wait_limit_ns)), int(skip_stage))
    if rc != 0:
        raise KernelError("stream_test_hooks: could not set the device words")


def stream_error() -> int:
    """Error word of the streaming kernels: 0, or (code << 16 | block) of a bounded wait that ran
    out (1: the producer waited for a free stage, 2: a consumer waited for data).  Reading clears it.
    Synchronises the device."""
    return int(_lib().kvcm_stream_error())


def qkv_rope_cache(x: torch.Tensor, w_qkv: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor,
                   inv_freq: torch.Tensor, slot_mapping: torch.Tensor, k_cache: torch.Tensor,
                   v_cache: torch.Tensor, nh: int, nkv: int, hd: int,
                   partials: Optional[torch.Tensor] = None, eps: float = 0.0) -> None:
    """Fused decode kernel: qkv product (M <= 16), rotate-half rotary encoding over the whole head,
    q into ``q_out`` [M, nh*hd], k (rotated) and v into the rows' cache page slots.  Gives the same
    bits as ``gemm_stream`` followed by ``rope_cache``.  With ``partials`` (float32 [tiles, 16] as
    ``gemm_stream_residual`` leaves them) row m of the product is first scaled by
    rsqrt(sum(partials[:, m]) / K + eps): ``x`` is then a normed row before its scale."""
    _cuda(x, w_qkv, q_out, positions, inv_freq, slot_mapping, k_cache, v_cache, partials)
    _need(partials is None or (partials.dtype == torch.float32 and partials.is_contiguous() and partials.dim() == 2
                               and partials.shape[1] == 16), "qkv_rope_cache: partials float32 [tiles, 16]")
    M, K = x.shape
    _need(w_qkv.shape == ((nh + 2 * nkv) * hd, K) and q_out.shape[0] == M and q_out.shape[1] >= nh * hd,
          "qkv_rope_cache: shapes")
    _need(x.dtype == w_qkv.dtype == q_out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16,
          "qkv_rope_cache: bfloat16 only")
    _need(x.stride(1) == 1 and w_qkv.stride(1) == 1 and q_out.stride(1) == 1 and k_cache.is_contiguous()
          and v_cache.is_contiguous(), "qkv_rope_cache: layout")
    _need(tuple(k_cache.shape[1:]) == (nkv, k_cache.shape[2], hd), "qkv_rope_cache: cache page shape")
    _need(positions.dtype == _I32 and slot_mapping.dtype == _I32 and positions.numel() >= M
          and slot_mapping.numel() >= M, "qkv_rope_cache: positions/slot_mapping int32 [M]")
    _need(inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == hd, "qkv_rope_cache: inv_freq float32 [hd/2]")
    rc = _lib().kvcm_qkv_rope_cache_scaled_bf16(_p(x), _p(partials) if partials is not None else None,
                                                partials.shape[0] if partials is not None else 0, ctypes.c_float(eps),
                                                _p(w_qkv), _p(q_out), M, K, x.stride(0), w_qkv.stride(0),
                                                q_out.stride(0), _p(positions), _p(inv_freq), _p(slot_mapping),
                                                _p(k_cache), _p(v_cache), nh, nkv, hd, k_cache.shape[2],
                                                sm_count(x.device), _stream())
    _check(rc, "qkv_rope_cache", f"(M={M}, K={K}, nh={nh}, nkv={nkv}, hd={hd})")


def gemm_stream_residual(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, partials: torch.Tensor,
                         h_out: Optional[torch.Tensor] = None, next_w: Optional[torch.Tensor] = None) -> None:
    """The product that ends a sublayer (M <= 16): resid[M,N] (float32, in place) += bfloat16(x @ w^T);
    partials[t, m] = the sum over columns 16t..16t+15 of the new resid[m]^2 (``partials`` float32
    [ceil(N/16), 16]); and with ``next_w`` (bfloat16 [N]) h_out[M,N] = bfloat16(next_w * resid): the row
    the next norm hands on before its scale, which the ``partials`` argument of ``qkv_rope_cache`` and
    ``gate_up_silu`` applies."""
    _cuda(x, w, resid, partials, h_out, next_w)
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and resid.shape == (M, N), "gemm_stream_residual: shapes")
    _need(x.dtype == w.dtype == torch.bfloat16 and resid.dtype == partials.dtype == torch.float32,
          "gemm_stream_residual: bfloat16 operands, float32 residual and partial sums")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and resid.stride(1) == 1, "gemm_stream_residual: rows must be dense")
    _need(partials.is_contiguous() and tuple(partials.shape) == ((N + 15) // 16, 16), "gemm_stream_residual: partials [ceil(N/16), 16]")
    _need((h_out is None) == (next_w is None), "gemm_stream_residual: h_out and next_w go together")
    if next_w is not None:
        _need(h_out.dtype == next_w.dtype == torch.bfloat16 and h_out.shape == (M, N) and h_out.stride(1) == 1
              and next_w.numel() == N and next_w.is_contiguous(), "gemm_stream_residual: h_out [M,N], next_w [N] bfloat16")
    rc = _lib().kvcm_gemm_stream_residual_bf16(_p(x), _p(w), _p(resid), _p(partials),
                                               _p(h_out) if h_out is not None else None,
                                               _p(next_w) if next_w is not None else None, M, N, K, x.stride(0),
                                               w.stride(0), resid.stride(0), h_out.stride(0) if h_out is not None else 0,
                                               sm_count(x.device), _stream())
    _check(rc, "gemm_stream_residual", f"(M={M}, N={N}, K={K})")


def qkv_rope_cache_supported(M: int, K: int, nh: int, nkv: int, hd: int) -> bool:
    return hd % 16 == 0 and bool(_lib().kvcm_gemm_stream_fused_supports(int(M), int((nh + 2 * nkv) * hd), int(K)))


def gate_up_silu(x: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor,
                 partials: Optional[torch.Tensor] = None, eps: float = 0.0) -> None:
    """Fused decode kernel: act[M, I] = silu(x Wg^T) * (x Wu^T), Wg/Wu the halves of w [2I, K].
    ``partials``: both products scaled per row first, as in ``qkv_rope_cache``."""
    _cuda(x, w_gate_up, act, partials)
    _need(partials is None or (partials.dtype == torch.float32 and partials.is_contiguous() and partials.dim() == 2
                               and partials.shape[1] == 16), "gate_up_silu: partials float32 [tiles, 16]")
    M, K = x.shape
    I = act.shape[1]
    _need(w_gate_up.shape == (2 * I, K) and act.shape[0] == M, "gate_up_silu: shapes")
    _need(x.dtype == w_gate_up.dtype == act.dtype == torch.bfloat16, "gate_up_silu: bfloat16 only")
    _need(x.stride(1) == 1 and w_gate_up.stride(1) == 1 and act.stride(1) == 1, "gate_up_silu: layout")
    rc = _lib().kvcm_gate_up_silu_scaled_bf16(_p(x), _p(partials) if partials is not None else None,
                                              partials.shape[0] if partials is not None else 0, ctypes.c_float(eps),
                                              _p(w_gate_up), _p(act), M, I, K, x.stride(0), w_gate_up.stride(0),
                                              act.stride(0), sm_count(x.device), _stream())
    _check(rc, "gate_up_silu", f"(M={M}, I={I}, K={K})")


def gate_up_silu_supported(M: int, I: int, K: int) -> bool:
    return I % 8 == 0 and bool(_lib().kvcm_gemm_stream_fused_supports(int(M), int(2 * I), int(K)))


def gate_up_silu_tcgen05(x: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor) -> None:
    """act[M, I] = silu(x Wg^T) * (x Wu^T) for many rows: the tcgen05 product with the activation in
    its epilogue (the roundings of the separate product and activation kernels); the [M, 2I]
    intermediate never goes to memory."""
    _cuda(x, w_gate_up, act)
    M, K = x.shape
    I = act.shape[1]
    _need(w_gate_up.shape == (2 * I, K) and act.shape[0] == M, "gate_up_silu_tcgen05: shapes")
    _need(x.dtype == w_gate_up.dtype == act.dtype == torch.bfloat16, "gate_up_silu_tcgen05: bfloat16 only")
    _need(x.stride(1) == 1 and w_gate_up.stride(1) == 1 and act.stride(1) == 1, "gate_up_silu_tcgen05: rows must be dense")
    rc = _lib().kvcm_gate_up_silu_tcgen05_bf16(_p(x), _p(w_gate_up), _p(act), M, I, K, x.stride(0),
                                               w_gate_up.stride(0), act.stride(0), _stream())
    _check(rc, "gate_up_silu_tcgen05", f"(M={M}, I={I}, K={K})")


def tcgen05_gemm_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """True when the tcgen05 kernel takes this product (bfloat16, K and row strides multiples of 8)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(_lib().kvcm_gemm_tcgen05_supports(x.shape[0], w.shape[0], x.shape[1], x.stride(0), w.stride(0))))


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> None:
    """y[M,N] = x[M,K] @ w[N,K]^T on the fifth-generation tensor cores (TMA tensor maps, tcgen05.mma
    with the accumulator in tensor memory).  bfloat16 operands; bfloat16 or float32 result."""
    _cuda(x, w, y)
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and y.shape == (M, N), "gemm_tcgen05: shapes")
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and y.dtype in (torch.bfloat16, torch.float32),
          "gemm_tcgen05: bfloat16 operands, bfloat16 or float32 result")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and y.stride(1) == 1, "gemm_tcgen05: rows must be dense")
    rc = _lib().kvcm_gemm_tcgen05_bf16(_p(x), _p(w), _p(y), M, N, K, x.stride(0), w.stride(0), y.stride(0),
                                       int(y.dtype == torch.float32), _stream())
    _check(rc, "gemm_tcgen05", f"(M={M}, N={N}, K={K})")


def splitk_gemm_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """True when the split-K tcgen05 kernel takes this product (up to 256 rows, bfloat16, K and row
    strides multiples of 8)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(_lib().kvcm_gemm_tcgen05_splitk_supports(x.shape[0], w.shape[0], x.shape[1], x.stride(0), w.stride(0))))


def gemm_tcgen05_splitk(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> None:
    """y[M,N] = x[M,K] @ w[N,K]^T for M <= 256 on the fifth-generation tensor cores with the operands
    swapped (128 weight rows are the tall operand) and K split over a thread-block cluster whose
    blocks add their partial sums through distributed shared memory.  bfloat16 operands; bfloat16 or
    float32 result."""
    _cuda(x, w, y)
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and y.shape == (M, N), "gemm_tcgen05_splitk: shapes")
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and y.dtype in (torch.bfloat16, torch.float32),
          "gemm_tcgen05_splitk: bfloat16 operands, bfloat16 or float32 result")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and y.stride(1) == 1, "gemm_tcgen05_splitk: rows must be dense")
    rc = _lib().kvcm_gemm_tcgen05_splitk_bf16(_p(x), _p(w), _p(y), M, N, K, x.stride(0), w.stride(0), y.stride(0),
                                              int(y.dtype == torch.float32), _stream())
    _check(rc, "gemm_tcgen05_splitk", f"(M={M}, N={N}, K={K})")


def splitk_error() -> int:
    """Error word of the split-K tcgen05 kernel: 0, or (code << 16 | block) of a bounded wait that
    ran out.  Reading clears it.  Synchronises the device."""
    return int(_lib().kvcm_gemm_tcgen05_splitk_error())


def pair_gemm_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """True when the two-SM tcgen05 kernel takes this product (bfloat16, K and row strides multiples of 8)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(_lib().kvcm_gemm_tcgen05_pair_supports(x.shape[0], w.shape[0], x.shape[1], x.stride(0), w.stride(0))))


_pair_workspaces: dict = {}


def _pair_workspace(device: torch.device, split: int):
    """Partial sums and flags of the two-SM kernel's split walk, one set per device (the kernel's
    launches on a device are expected on one stream at a time).  (None, None, 0) without it."""
    if split == 0:
        return None, None, 0
    key = torch.device(device).index or 0
    ws = _pair_workspaces.get(key)
    if ws is None:
        if torch.cuda.is_current_stream_capturing():
            return None, None, 0
        slots = int(_lib().kvcm_gemm_tcgen05_pair_capacity())
        if slots <= 0:
            return None, None, 0
        part = torch.empty(slots * int(_lib().kvcm_gemm_tcgen05_pair_slot_floats()), dtype=torch.float32, device=device)
        flag = torch.zeros(slots * int(_lib().kvcm_gemm_tcgen05_pair_slot_flags()), dtype=torch.int32, device=device)
        ws = _pair_workspaces[key] = (part, flag, slots)
    return ws


def gemm_tcgen05_pair(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, bn: int = 0, band: int = 0,
                      split: int = -1) -> None:
    """y[M,N] = x[M,K] @ w[N,K]^T with 256 x bn tiles computed by pairs of SMs (tcgen05.mma.cta_group::2:
    each block of a pair loads half of the tile's rows of w).  bn: tile width, band: row tiles walked
    together; 0 = chosen by the kernel's host side.  split: 1 = equal shares of k-steps for every
    pair (partial sums through a workspace), 0 = whole tiles, -1 = chosen by the host side.
    bfloat16 operands; bfloat16 or float32 result."""
    _cuda(x, w, y)
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and y.shape == (M, N), "gemm_tcgen05_pair: shapes")
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and y.dtype in (torch.bfloat16, torch.float32),
          "gemm_tcgen05_pair: bfloat16 operands, bfloat16 or float32 result")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and y.stride(1) == 1, "gemm_tcgen05_pair: rows must be dense")
    part, flag, slots = _pair_workspace(x.device, split)
    rc = _lib().kvcm_gemm_tcgen05_pair_bf16(_p(x), _p(w), _p(y), M, N, K, x.stride(0), w.stride(0), y.stride(0),
                                            int(y.dtype == torch.float32), int(bn), int(band), int(split),
                                            _p(part) if part is not None else None,
                                            _p(flag) if flag is not None else None, slots, _stream())
    _check(rc, "gemm_tcgen05_pair", f"(M={M}, N={N}, K={K}, bn={bn}, split={split})")


def gate_up_silu_tcgen05_pair(x: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor, bn: int = 0,
                              band: int = 0, split: int = -1) -> None:
    """act[M, I] = silu(x Wg^T) * (x Wu^T) on pairs of SMs: one block of a pair loads the tile's gate
    rows, the other its up rows, and the epilogue applies the activation (the roundings of the
    separate product and activation kernels)."""
    _cuda(x, w_gate_up, act)
    M, K = x.shape
    I = act.shape[1]
    _need(w_gate_up.shape == (2 * I, K) and act.shape[0] == M, "gate_up_silu_tcgen05_pair: shapes")
    _need(x.dtype == w_gate_up.dtype == act.dtype == torch.bfloat16, "gate_up_silu_tcgen05_pair: bfloat16 only")
    _need(x.stride(1) == 1 and w_gate_up.stride(1) == 1 and act.stride(1) == 1, "gate_up_silu_tcgen05_pair: rows must be dense")
    part, flag, slots = _pair_workspace(x.device, split)
    rc = _lib().kvcm_gate_up_silu_tcgen05_pair_bf16(_p(x), _p(w_gate_up), _p(act), M, I, K, x.stride(0),
                                                    w_gate_up.stride(0), act.stride(0), int(bn), int(band), int(split),
                                                    _p(part) if part is not None else None,
                                                    _p(flag) if flag is not None else None, slots, _stream())
    _check(rc, "gate_up_silu_tcgen05_pair", f"(M={M}, I={I}, K={K}, bn={bn}, split={split})")


def pair_error() -> int:
    """Error word of the two-SM tcgen05 kernel: 0, or (code << 16 | block) of a bounded wait that ran
    out (1: a TMA thread waited for a free stage, 2: the MMA thread waited for data, 3: an epilogue
    waited for the accumulator, 4: the MMA thread waited for the epilogues, 5: an epilogue waited for
    another pair's partial sums).  Reading clears it.
    Synchronises the device."""
    return int(_lib().kvcm_gemm_tcgen05_pair_error())


def tcgen05_error() -> int:
    """Error word of the tcgen05 kernel: 0, or (code << 16 | block) of a bounded wait that ran out
    (1: the TMA thread waited for a free stage, 2: the MMA thread waited for data, 3: the epilogue
    waited for the accumulator).  Reading clears it.  Synchronises the device."""
    return int(_lib().kvcm_tcgen05_error())


# ------------------------------------------------------------------ the step's forward pass from C++

FORWARD_MAX_GROUPS = 4


class ForwardLayer(ctypes.Structure):
    """One call site of the run order (csrc/cuda/step_forward.cu: KvcmForwardLayer)."""
    _fields_ = [("w_qkv", ctypes.c_void_p), ("w_o", ctypes.c_void_p), ("w_gate_up", ctypes.c_void_p),
                ("w_down", ctypes.c_void_p), ("norm1", ctypes.c_void_p), ("norm2", ctypes.c_void_p),
                ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p),
                ("eps1", ctypes.c_float), ("eps2", ctypes.c_float),
                ("group", ctypes.c_int), ("window", ctypes.c_int), ("writes", ctypes.c_int), ("num_pages", ctypes.c_int)]


class ForwardArgs(ctypes.Structure):
    """The argument block of ``kvcm_forward`` (csrc/cuda/step_forward.cu: KvcmForwardArgs)."""
    _fields_ = [
        ("layers", ctypes.c_void_p), ("embed", ctypes.c_void_p), ("final_norm", ctypes.c_void_p),
        ("lm_head", ctypes.c_void_p), ("inv_freq", ctypes.c_void_p),
        ("tokens", ctypes.c_void_p), ("positions", ctypes.c_void_p), ("row_seq", ctypes.c_void_p),
        ("seq_q_start", ctypes.c_void_p), ("seq_q_len", ctypes.c_void_p), ("seq_ctx_len", ctypes.c_void_p),
        ("tile_seq", ctypes.c_void_p), ("tile_q0", ctypes.c_void_p), ("logit_rows", ctypes.c_void_p),
        ("group_tables", ctypes.c_void_p * FORWARD_MAX_GROUPS), ("group_slots", ctypes.c_void_p * FORWARD_MAX_GROUPS),
        ("x", ctypes.c_void_p), ("h", ctypes.c_void_p), ("qkv", ctypes.c_void_p), ("attn", ctypes.c_void_p),
        ("proj", ctypes.c_void_p), ("gate_up", ctypes.c_void_p), ("act", ctypes.c_void_p), ("h_last", ctypes.c_void_p),
        ("logits", ctypes.c_void_p), ("attn_scratch", ctypes.c_void_p), ("lib_workspace", ctypes.c_void_p),
        ("norm_partials", ctypes.c_void_p), ("rope_table", ctypes.c_void_p),
        ("attn_scratch_floats", ctypes.c_longlong), ("lib_workspace_bytes", ctypes.c_longlong),
        ("norm_partials_floats", ctypes.c_longlong), ("rope_table_floats", ctypes.c_longlong),
        ("num_layers", ctypes.c_int), ("f32", ctypes.c_int), ("H", ctypes.c_int), ("I", ctypes.c_int),
        ("nh", ctypes.c_int), ("nkv", ctypes.c_int), ("hd", ctypes.c_int), ("V", ctypes.c_int),
        ("block_size", ctypes.c_int), ("max_blocks", ctypes.c_int), ("sm_count", ctypes.c_int),
        ("rows", ctypes.c_int), ("seqs", ctypes.c_int), ("decode_seqs", ctypes.c_int), ("prefill_tiles", ctypes.c_int),
        ("tile_rows", ctypes.c_int), ("max_decode_ctx", ctypes.c_int), ("num_logits", ctypes.c_int),
        ("reserved", ctypes.c_int),
        ("final_eps", ctypes.c_float), ("scale", ctypes.c_float),
    ]


def forward_layouts_match() -> bool:
    lib = _lib()
    return (ctypes.sizeof(ForwardArgs) == int(lib.kvcm_forward_args_bytes())
            and ctypes.sizeof(ForwardLayer) == int(lib.kvcm_forward_layer_bytes()))


_forward_launches = ctypes.c_int(0)


def forward(args: ForwardArgs) -> int:
    """The whole forward pass of a step launched from C++ (csrc/cuda/step_forward.cu); returns the
    number of kernel launches it made.  The caller owns every buffer the block names."""
    global _launches
    rc = _lib().kvcm_forward(ctypes.byref(args), ctypes.byref(_forward_launches), _stream())
    n = int(_forward_launches.value)
    _launches += n
    if _profile is not None:
        profile_mark("forward (whole step)")
    if rc == 0:
        return n
    if rc == _ERR_UNSUPPORTED:
        raise KernelError(f"forward: sizes not supported (rows {args.rows}, hidden {args.H}, heads {args.nh}/{args.nkv} "
                          f"of {args.hd})")
    raise KernelError(f"forward: error {rc} at a launch (rows {args.rows})")


# ------------------------------------------------ kernels around an output-normed residual stream

def _ll(v) -> ctypes.c_longlong:
    return ctypes.c_longlong(int(v))


def embed_sum(ids: torch.Tensor, prev: Optional[torch.Tensor], positions: torch.Tensor, table: torch.Tensor,
              pair: Optional[torch.Tensor], place: Optional[torch.Tensor], x: torch.Tensor,
              h: Optional[torch.Tensor], buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0) -> None:
    """x[t] = table[id] + pair[(prev*mul_prev + id*mul_cur) % buckets, or row `buckets` without an earlier
    token] + place[position]; x float32 [T, H]; ``h`` (optional) the same rows in the tables' dtype."""
    _cuda(ids, prev, positions, table, pair, place, x, h)
    T, H = x.shape
    _need(ids.dtype == _I32 and positions.dtype == _I32 and ids.numel() >= T and positions.numel() >= T,
          "embed_sum: ids/positions int32 [T]")
    _need(x.dtype == torch.float32 and x.is_contiguous() and table.is_contiguous() and table.shape[1] == H, "embed_sum: layout")
    for t in (pair, place):
        _need(t is None or (t.dtype == table.dtype and t.is_contiguous() and t.shape[1] == H), "embed_sum: tables differ")
    _need(pair is None or (prev is not None and prev.dtype == _I32 and prev.numel() >= T and pair.shape[0] == buckets + 1),
          "embed_sum: the pair table needs buckets + 1 rows and the rows' previous tokens")
    _need(h is None or (h.dtype == table.dtype and h.is_contiguous() and h.shape == x.shape), "embed_sum: h")
    fn = getattr(_lib(), "kvcm_embed_sum_" + _suffix(table))
    _check(fn(_p(ids), _p(prev), _p(positions), _p(table), _p(pair), _p(place), _p(x), _p(h), T, H, table.shape[0],
              int(buckets), _ll(mul_prev), _ll(mul_cur), place.shape[0] if place is not None else 0, _stream()), "embed_sum")


def rms_scale_add(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, h: Optional[torch.Tensor],
                  eps: float, mult: float) -> None:
    """x += mult * weight * y / sqrt(mean(y^2) + eps) row by row (x float32, y float32 or the storage
    dtype); ``h`` (optional, storage dtype) receives the new rows of x."""
    _cuda(x, y, weight, h)
    T, H = x.shape
    _need(x.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and y.shape == x.shape
          and weight.numel() == H, "rms_scale_add: shapes")
    store = h.dtype if h is not None else (y.dtype if y.dtype != torch.float32 else weight.dtype)
    _need(y.dtype in (torch.float32, store) and weight.dtype in (torch.float32, store), "rms_scale_add: dtypes")
    _need(h is None or (h.is_contiguous() and h.shape == x.shape), "rms_scale_add: h")
    fn = getattr(_lib(), "kvcm_rms_scale_add_" + _SUFFIX[store])
    _check(fn(_p(x), _p(y), int(y.dtype == torch.float32), _p(weight), int(weight.dtype == torch.float32), _p(h),
              T, H, ctypes.c_float(eps), ctypes.c_float(mult), _stream()), "rms_scale_add", f"(hidden={H})")


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(x, out)
    _need(x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and x.shape == out.shape, "cast_rows: layout")
    fn = getattr(_lib(), "kvcm_cast_rows_" + _suffix(out))
    _check(fn(_p(x), _p(out), _ll(x.numel()), _stream()), "cast_rows")


def gemm_plain_batched(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> None:
    """y[m, b, :] = x[m, b, :] @ w[b]^T for every b: x [M, B, K] (rows and heads may be strided, K dense),
    w [B, N, K] contiguous, y [M, B, N] (K-dense too).  Plain kernel, float accumulation in a fixed order."""
    _cuda(x, w, y)
    M, B, K = x.shape
    N = w.shape[1]
    _need(w.shape == (B, N, K) and w.is_contiguous() and y.shape == (M, B, N), "gemm_plain_batched: shapes")
    _need(x.stride(2) == 1 and y.stride(2) == 1 and x.dtype == w.dtype == y.dtype, "gemm_plain_batched: layout")
    fn = getattr(_lib(), "kvcm_gemm_plain_batched_" + _suffix(x))
    _check(fn(_p(x), _p(w), _p(y), M, N, K, x.stride(0), K, y.stride(0), B, _ll(x.stride(1)), _ll(N * K),
              _ll(y.stride(1)), _stream()), "gemm_plain_batched")


# ------------------------------------------------------------------------ the gated delta rule

def delta_scan_max_dk() -> int:
    return int(_lib().kvcm_delta_scan_max_dk())


def delta_conv(proj: torch.Tensor, conv_w: torch.Tensor, state: torch.Tensor, conv_off: int, ctx,
               out: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
    """Causal convolution over time + SiLU of the first ``channels`` columns of ``proj`` into float32
    ``out`` [T, channels]; earlier inputs come from (and the newest go to) the requests' state rows."""
    _cuda(proj, conv_w, state, out, bias)
    T, C = out.shape
    taps = conv_w.shape[1]
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == C), "delta_conv: bias float32 [channels]")
    _need(conv_w.dtype == torch.float32 and conv_w.is_contiguous() and conv_w.shape[0] == C, "delta_conv: taps [channels, taps] float32")
    _need(out.dtype == torch.float32 and out.is_contiguous() and proj.stride(1) == 1 and proj.shape[1] >= C, "delta_conv: layout")
    _need(state.dtype == torch.float32 and state.is_contiguous() and state.dim() == 2
          and state.shape[1] >= conv_off + (taps - 1) * C, "delta_conv: state rows too short")
    fn = getattr(_lib(), "kvcm_delta_conv_" + _suffix(proj))
    _check(fn(_p(proj), proj.stride(0), _p(conv_w), taps, _p(state), _ll(state.stride(0)), _ll(conv_off), _p(ctx.row_seq),
              _p(ctx.seq_q_start), _p(ctx.seq_q_len), _p(ctx.seq_state_slot), _p(out), T, ctx.seqs, C, _p(bias), _stream()), "delta_conv")
    if taps > 1 and T != ctx.seqs:
        global _launches
        _launches += 1                      # the state update (a kernel of its own unless every request brings one row)


def delta_prepare(qkv: torch.Tensor, ba: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
                  heads: int, qk_heads: int, dk: int) -> None:
    """In place: query and key heads of ``qkv`` to unit length (queries also times dk^-1/2);
    ``ba`` = [b | a] becomes [sigmoid(b) | exp(-exp(A_log) softplus(a + dt_bias))]."""
    _cuda(qkv, ba, a_log, dt_bias)
    _need(all(t.dtype == torch.float32 and t.is_contiguous() for t in (qkv, ba, a_log, dt_bias)), "delta_prepare: float32")
    _need(ba.shape == (qkv.shape[0], 2 * heads) and a_log.numel() == heads and dt_bias.numel() == heads
          and qkv.shape[1] >= 2 * qk_heads * dk, "delta_prepare: shapes")
    _check(_lib().kvcm_delta_prepare(_p(qkv), qkv.shape[1], _p(ba), _p(a_log), _p(dt_bias), qkv.shape[0], heads, qk_heads,
                                     dk, _stream()), "delta_prepare")


def delta_scan(qkv: torch.Tensor, bg: torch.Tensor, state: torch.Tensor, ctx, out: torch.Tensor,
               heads: int, qk_heads: int, dk: int, dv: int) -> None:
    """The recurrence over every request's rows of the step, from and into its state row."""
    _cuda(qkv, bg, state, out)
    _need(all(t.dtype == torch.float32 and t.is_contiguous() for t in (qkv, bg, state, out)), "delta_scan: float32")
    _need(qkv.shape[1] == 2 * qk_heads * dk + heads * dv and out.shape == (qkv.shape[0], heads * dv)
          and state.shape[1] >= heads * dk * dv, "delta_scan: shapes")
    _check(_lib().kvcm_delta_scan(_p(qkv), qkv.shape[1], _p(bg), _p(state), _ll(state.stride(0)), _p(ctx.seq_q_start),
                                  _p(ctx.seq_q_len), _p(ctx.seq_state_slot), _p(out), qkv.shape[0], ctx.seqs, heads, qk_heads, dk, dv,
                                  _stream()), "delta_scan", f"(dk={dk}, dv={dv})")


def gated_rms(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, heads: int,
              dv: int, eps: float) -> None:
    """out[t, h, :] = o[t, h, :] / rms * weight * silu(gate[t, h, :]); o float32, gate/out storage dtype."""
    _cuda(o, gate, weight, out)
    T = o.shape[0]
    _need(o.dtype == torch.float32 and o.is_contiguous() and o.shape == (T, heads * dv) and out.is_contiguous()
          and out.shape == o.shape and gate.stride(1) == 1 and gate.shape[1] >= heads * dv and gate.dtype == out.dtype
          and weight.dtype == torch.float32 and weight.numel() == dv, "gated_rms: layout")
    fn = getattr(_lib(), "kvcm_gated_rms_" + _suffix(out))
    _check(fn(_p(o), _p(gate), gate.stride(0), _p(weight), _p(out), T, heads, dv, ctypes.c_float(eps), _stream()), "gated_rms")


# ----------------------------------------------------------------------------- latent cache

def latent_norm_cache(v: torch.Tensor, weight: torch.Tensor, slot_mapping: torch.Tensor, cache: torch.Tensor,
                      eps: float) -> None:
    """cache[slot of row] = weight * v[row] / sqrt(mean(v[row]^2) + eps); cache [pages, 1, page, width]."""
    _cuda(v, weight, slot_mapping, cache)
    T, R = v.shape
    _need(v.stride(1) == 1 and v.dtype == cache.dtype and cache.is_contiguous() and cache.shape[1] == 1
          and cache.shape[3] == R, "latent_norm_cache: layout")
    _need(weight.dtype == torch.float32 and weight.numel() == R and slot_mapping.dtype == _I32
          and slot_mapping.numel() >= T, "latent_norm_cache: weight float32 [width], slots int32 [T]")
    fn = getattr(_lib(), "kvcm_latent_norm_cache_" + _suffix(v))
    _check(fn(_p(v), v.stride(0), _p(weight), _p(slot_mapping), _p(cache), T, R, ctypes.c_float(eps), _stream()),
           "latent_norm_cache")


# ---------------------------------------------------------------------------- routed experts

def moe_route(h: torch.Tensor, router: torch.Tensor, experts: int, groups: int, keep: int, top: int, scale: float,
              idx: torch.Tensor, wt: torch.Tensor, gate: Optional[torch.Tensor], scores: str = "softmax",
              correction: Optional[torch.Tensor] = None, group_top: int = 1) -> None:
    """Per row: float32 router logits, scores (``scores``: "softmax" over all experts or "sigmoid" of each
    logit), group-limited choice of ``top`` experts; ``idx`` int32 [T, top], ``wt`` float32 [T, top] =
    score * scale; ``gate`` float32 [T] = sigmoid of the logit of the router matrix's extra row (row
    ``experts``).  ``correction`` (float32 [experts]) is added to the scores for the choice only;
    ``group_top``: a group's score is the sum of its 1 or 2 largest choice scores."""
    _cuda(h, router, idx, wt, gate, correction)
    _need(scores in ("softmax", "sigmoid") and group_top in (1, 2), "moe_route: scores 'softmax' | 'sigmoid', group_top 1 | 2")
    _need(correction is None or (correction.dtype == torch.float32 and correction.is_contiguous() and correction.numel() == experts),
          "moe_route: correction float32 [experts]")
    T, D = h.shape
    _need(h.stride(1) == 1 and router.is_contiguous() and router.shape == (experts + (gate is not None), D)
          and router.dtype in (torch.float32, h.dtype), "moe_route: router [experts (+1), width]")
    _need(idx.dtype == _I32 and idx.is_contiguous() and idx.shape == (T, top) and wt.dtype == torch.float32
          and wt.is_contiguous() and wt.shape == (T, top), "moe_route: outputs")
    _need(gate is None or (gate.dtype == torch.float32 and gate.numel() >= T), "moe_route: gate float32 [T]")
    fn = getattr(_lib(), "kvcm_moe_route_" + _suffix(h))
    _check(fn(_p(h), h.stride(0), _p(router), int(router.dtype == torch.float32), T, D, experts, groups, keep, top,
              ctypes.c_float(scale), int(gate is not None), int(scores == "sigmoid"), _p(correction), int(group_top),
              _p(idx), _p(wt), _p(gate), _stream()), "moe_route",
           f"(experts={experts}, groups={groups}, keep={keep}, top={top})")


def moe_work_ints(rows: int, top: int, experts: int) -> int:
    return int(_lib().kvcm_moe_work_ints(int(rows), int(top), int(experts)))


def moe_tcgen05_supported(expert_ff: int, hidden: int) -> bool:
    return bool(_lib().kvcm_moe_tcgen05_supports(int(expert_ff), int(hidden)))


def moe_tcgen05_error() -> int:
    """Error word of the experts' tensor-core products: 0, or (code << 16 | block) of a bounded wait
    that ran out.  Reading clears it.  Synchronises the device."""
    return int(_lib().kvcm_moe_tcgen05_error())


def moe_experts(h: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, idx: torch.Tensor,
                work: torch.Tensor, act: torch.Tensor, y: torch.Tensor, xs: Optional[torch.Tensor] = None) -> None:
    """y[place of (t, k)] = expert idx[t, k] applied to h[t] (float32 [T * top, D], in the order of the
    pairs sorted by expert; ``work`` keeps every pair's place for ``moe_combine``); w_gate_up
    [E, 2F, D] (gate rows before up rows), w_down [E, D, F]; act [T * top, F] and work int32 are
    scratch.  With ``xs`` (bfloat16 [T * top, D] scratch) the products run on the tensor cores."""
    _cuda(h, w_gate_up, w_down, idx, work, act, y, xs)
    T, D = h.shape
    top = idx.shape[1]
    E, F2, _ = w_gate_up.shape
    F = F2 // 2
    _need(w_gate_up.is_contiguous() and w_down.is_contiguous() and w_gate_up.shape == (E, 2 * F, D)
          and w_down.shape == (E, D, F) and w_gate_up.dtype == h.dtype == w_down.dtype == act.dtype, "moe_experts: weights")
    _need(h.stride(1) == 1 and act.is_contiguous() and act.shape == (T * top, F) and y.dtype == torch.float32
          and y.is_contiguous() and y.shape == (T * top, D), "moe_experts: buffers")
    _need(work.dtype == _I32 and work.numel() >= moe_work_ints(T, top, E), "moe_experts: work too small")
    global _launches
    if xs is not None:
        _need(h.dtype == torch.bfloat16 and xs.dtype == torch.bfloat16 and xs.is_contiguous() and xs.shape == (T * top, D),
              "moe_experts: the tensor-core form takes bfloat16 rows and a [pairs, width] scratch")
        _check(_lib().kvcm_moe_experts_tc_bf16(_p(h), h.stride(0), _p(w_gate_up), _p(w_down), _p(idx), T, top, E, F, D,
                                               _p(work), _p(xs), _p(act), _p(y), _stream()),
               "moe_experts_tcgen05", f"(experts={E}, ff={F})")
        _launches += 3                      # sort, gather, gate/up, down
        return
    fn = getattr(_lib(), "kvcm_moe_experts_" + _suffix(h))
    _check(fn(_p(h), h.stride(0), _p(w_gate_up), _p(w_down), _p(idx), T, top, E, F, D, _p(work), _p(act), _p(y), _stream()),
           "moe_experts", f"(experts={E}, ff={F})")
    _launches += 2                          # sort, gate/up, down


def moe_combine(y: torch.Tensor, work: torch.Tensor, wt: torch.Tensor, experts: int, shared_y: Optional[torch.Tensor],
                gate: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[t] = sum_k wt[t, k] * y[place of (t, k)] + gate[t] * shared_y[t]; all float32; ``work`` is the
    scratch that ``moe_experts`` filled."""
    _cuda(y, work, wt, shared_y, gate, out)
    T, D = out.shape
    top = wt.shape[1]
    _need(all(t is None or (t.dtype == torch.float32 and t.is_contiguous()) for t in (y, wt, shared_y, gate, out)),
          "moe_combine: float32")
    _need(y.shape == (T * top, D) and (shared_y is None or shared_y.shape == (T, D)) and work.dtype == _I32, "moe_combine: shapes")
    _check(_lib().kvcm_moe_combine(_p(y), _p(work), _p(wt), top, int(experts), _p(shared_y), _p(gate), _p(out), T, D,
                                   _stream()), "moe_combine")


# ------------------------------------------------- recurrences beside the head-wise delta rule

SCAN_DELTA, SCAN_DELTA_CHANNEL, SCAN_LINEAR, SCAN_LINEAR_CHANNEL = 0, 1, 2, 3


def state_scan(mode: int, qkv: torch.Tensor, bases, beta: Optional[torch.Tensor], g: Optional[torch.Tensor],
               gd: Optional[torch.Tensor], state: torch.Tensor, ctx, out: torch.Tensor, heads: int, qk_heads: int,
               dk: int, dv: int) -> None:
    """The matrix-state recurrences over every request's rows of the step, from and into its state row
    (csrc/cuda/delta_rule.cu).  ``bases`` = where a row's q, k and v start; ``beta`` [T, >= heads] (a view
    with a row stride is fine), ``g`` likewise (one decay per head) or ``gd`` [T, heads*dk] (one per head
    and key channel).  ``beta`` may be None for SCAN_LINEAR_CHANNEL (it then counts as one)."""
    _cuda(qkv, beta, g, gd, state, out)
    _need(all(t is None or t.dtype == torch.float32 for t in (qkv, beta, g, gd, state, out)), "state_scan: float32")
    _need(beta is not None or mode == SCAN_LINEAR_CHANNEL, "state_scan: beta")
    _need(qkv.is_contiguous() and out.is_contiguous() and state.is_contiguous() and (beta is None or beta.stride(1) == 1)
          and (g is None or g.stride(1) == 1) and (gd is None or (gd.is_contiguous() and gd.shape == (qkv.shape[0], heads * dk))),
          "state_scan: layout")
    qb, kb, vb = (int(b) for b in bases)
    C = qkv.shape[1]
    _need(max(qb, kb) + qk_heads * dk <= C and vb + heads * dv <= C and out.shape == (qkv.shape[0], heads * dv)
          and state.shape[1] >= heads * dk * dv and (beta is None or beta.shape[1] >= heads), "state_scan: shapes")
    _check(_lib().kvcm_state_scan(int(mode), _p(qkv), C, qb, kb, vb, _p(beta), beta.stride(0) if beta is not None else 0, _p(g),
                                  g.stride(0) if g is not None else 0, _p(gd), _p(state), _ll(state.stride(0)),
                                  _p(ctx.seq_q_start), _p(ctx.seq_q_len), _p(ctx.seq_state_slot), _p(out), qkv.shape[0],
                                  ctx.seqs, heads, qk_heads, dk, dv, _stream()), "state_scan", f"(mode={mode}, dk={dk}, dv={dv})")


def delta_prepare_channel(qkv: torch.Tensor, b: torch.Tensor, beta: torch.Tensor, a: torch.Tensor, a_log: torch.Tensor,
                          dt_bias: torch.Tensor, heads: int, qk_heads: int, dk: int) -> None:
    """In place: query and key heads of ``qkv`` to unit length (queries also times dk^-1/2); ``beta`` =
    sigmoid(b) (b [T, heads] in the storage dtype, any row stride); ``a`` [T, heads*dk] float32 becomes the
    decays exp(-exp(A_log[head]) softplus(a + dt_bias))."""
    _cuda(qkv, b, beta, a, a_log, dt_bias)
    T = qkv.shape[0]
    _need(all(t.dtype == torch.float32 and t.is_contiguous() for t in (qkv, beta, a, a_log, dt_bias)), "delta_prepare_channel: float32")
    _need(b.stride(1) == 1 and b.shape == (T, heads) and beta.shape == (T, heads) and a.shape == (T, heads * dk)
          and a_log.numel() == heads and dt_bias.numel() == heads * dk and qkv.shape[1] >= 2 * qk_heads * dk,
          "delta_prepare_channel: shapes")
    fn = getattr(_lib(), "kvcm_delta_prepare_channel_" + _suffix(b))
    _check(fn(_p(qkv), qkv.shape[1], _p(b), b.stride(0), _p(beta), _p(a), _p(a_log), _p(dt_bias), T, heads, qk_heads, dk,
              _stream()), "delta_prepare_channel")


def ssm_prepare(raw: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, out: torch.Tensor, heads: int) -> None:
    """out [T, 2*heads] float32 = [softplus(raw + dt_bias) | exp(-exp(A_log) * that)]; raw [T, heads] storage dtype."""
    _cuda(raw, a_log, dt_bias, out)
    T = raw.shape[0]
    _need(raw.stride(1) == 1 and raw.shape[1] == heads and out.dtype == torch.float32 and out.is_contiguous()
          and out.shape == (T, 2 * heads) and a_log.dtype == torch.float32 and dt_bias.dtype == torch.float32
          and a_log.numel() == heads and dt_bias.numel() == heads, "ssm_prepare: layout")
    fn = getattr(_lib(), "kvcm_ssm_prepare_" + _suffix(raw))
    _check(fn(_p(raw), raw.stride(0), _p(a_log), _p(dt_bias), _p(out), T, heads, _stream()), "ssm_prepare")


def group_rms_gate(o: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, group: int, eps: float,
                   gate_first: bool, act: str, skip: Optional[torch.Tensor] = None,
                   skip_coef: Optional[torch.Tensor] = None, head: int = 1) -> None:
    """Norm in groups of ``group`` neighbouring elements with a gate ``act`` ('silu' | 'sigmoid') of z before or
    after it; ``weight`` is indexed modulo its length; optional skip term ``skip_coef[i // head] * skip[:, i]``
    added to o first.  o/skip float32, z/out storage dtype (z and skip may have a row stride)."""
    _cuda(o, z, weight, out, skip, skip_coef)
    T, n = o.shape
    _need(o.dtype == torch.float32 and o.is_contiguous() and out.is_contiguous() and out.shape == o.shape
          and z.stride(1) == 1 and z.shape[1] >= n and z.dtype == out.dtype and weight.dtype == torch.float32
          and weight.is_contiguous() and n % group == 0, "group_rms_gate: layout")
    _need((skip is None) == (skip_coef is None), "group_rms_gate: skip and its coefficients come together")
    if skip is not None:
        _need(skip.dtype == torch.float32 and skip.stride(1) == 1 and skip.shape[1] >= n and skip_coef.dtype == torch.float32
              and skip_coef.is_contiguous() and skip_coef.numel() * head >= n, "group_rms_gate: skip layout")
    fn = getattr(_lib(), "kvcm_group_rms_gate_" + _suffix(out))
    _check(fn(_p(o), _p(z), z.stride(0), _p(skip), skip.stride(0) if skip is not None else 0, _p(skip_coef), int(head),
              _p(weight), weight.numel(), _p(out), T, n, int(group), int(bool(gate_first)), {"silu": 0, "sigmoid": 1}[act],
              ctypes.c_float(eps), _stream()), "group_rms_gate")


# ------------------------------------------------------- blocks with one norm and summed sublayers

def dyt_norm(x: torch.Tensor, pending, weight: torch.Tensor, bias: torch.Tensor, alpha: torch.Tensor,
             out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """x += sum of scale * tensor over ``pending`` (up to three (float32 tensor, scale) pairs; with ``rows``
    the sum is formed for the gathered rows only and x is left alone), then
    out = tanh(alpha * x) * weight + bias.  weight/bias float32 [H], alpha float32 [1] on the device."""
    pend = list(pending or [])
    _need(len(pend) <= 3, "dyt_norm: at most three pending outputs")
    _cuda(x, weight, bias, alpha, out, rows, *[t for t, _ in pend])
    H = x.shape[1]
    n = out.shape[0]
    _need(x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and out.shape[1] == H, "dyt_norm: x float32 [T,H]")
    _need(all(t.dtype == torch.float32 and t.is_contiguous() and t.numel() >= H for t in (weight, bias))
          and alpha.dtype == torch.float32 and alpha.numel() == 1, "dyt_norm: weight/bias/alpha float32")
    for t, _ in pend:
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.shape == x.shape, "dyt_norm: pending float32 like x")
    if rows is None:
        _need(n == x.shape[0], "dyt_norm: out rows != x rows")
    else:
        _need(rows.dtype == _I32 and rows.numel() >= n, "dyt_norm: rows int32 [n]")
    pend += [(None, 0.0)] * (3 - len(pend))
    fn = getattr(_lib(), "kvcm_dyt_norm_" + _suffix(out))
    _check(fn(_p(x), _p(pend[0][0]), ctypes.c_float(pend[0][1]), _p(pend[1][0]), ctypes.c_float(pend[1][1]),
              _p(pend[2][0]), ctypes.c_float(pend[2][1]), _p(weight), _p(bias), _p(alpha), _p(out), _p(rows), n, H,
              _stream()), "dyt_norm")


def relu_sq(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = max(x, 0)^2, elementwise, in the storage dtype."""
    _cuda(x, out)
    _need(x.is_contiguous() and out.is_contiguous() and x.shape == out.shape and x.dtype == out.dtype, "relu_sq: layout")
    fn = getattr(_lib(), "kvcm_relu_sq_" + _suffix(x))
    _check(fn(_p(x), _p(out), _ll(x.numel()), _stream()), "relu_sq")


def attn_prepare(proj: torch.Tensor, bias: Optional[torch.Tensor], wq: Optional[torch.Tensor], wk: Optional[torch.Tensor],
                 positions: torch.Tensor, inv_freq: Optional[torch.Tensor], rot: int, head_norm: bool, eps: float,
                 v_keep: Optional[torch.Tensor], v_first: Optional[torch.Tensor], lam: Optional[torch.Tensor],
                 slot_mapping: Optional[torch.Tensor], q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 nh: int, nkv: int, dk: int, dv: int, interleaved: bool = False,
                 v_inv_freq: Optional[torch.Tensor] = None, maps: int = 1) -> None:
    """From the float32 q|k|v projection of a step's rows to the attention kernel's inputs: optional bias,
    optional norm over the whole q and k projections (weights wq, wk), rotation of the first ``rot``
    dimensions of every head, optional per-head norm without weights, optional mixing of the values with
    ``v_first`` by ``lam``; q to ``q_out`` [T, nh*HD] and k, v to the rows' page slots, padded with zeros to the
    cache's head size HD (csrc/cuda/attn_prepare.cu).  ``interleaved``: rotary pairs (2i, 2i+1) instead of
    (i, i + rot/2); ``v_inv_freq`` (float32 [dv/2]): the values too are turned by their position, over all dv.
    ``maps`` > 1: every q and k head holds that many score maps of ``dk`` elements side by side; ``q_out`` is
    [T, nh*maps*HD], one padded head per map with the map at its own place, and a key head caches its maps in a row."""
    _cuda(proj, bias, wq, wk, positions, inv_freq, v_keep, v_first, lam, slot_mapping, q_out, k_cache, v_cache, v_inv_freq)
    _need(v_inv_freq is None or (v_inv_freq.dtype == torch.float32 and v_inv_freq.is_contiguous() and v_inv_freq.numel() * 2 == dv),
          "attn_prepare: v_inv_freq float32 [dv/2]")
    T = q_out.shape[0]
    HD, B = k_cache.shape[3], k_cache.shape[2]
    n = (nh + nkv) * maps * dk + nkv * dv
    _need(maps >= 1 and (maps == 1 or wq is None), "attn_prepare: several maps go without the whole-projection norm")
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[1] >= n and proj.shape[0] >= T, "attn_prepare: proj float32 [T, q|k|v]")
    for t, m in ((bias, n), (wq, nh * maps * dk), (wk, nkv * maps * dk), (lam, 1)):
        _need(t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == m), "attn_prepare: float32 vectors")
    _need((wq is None) == (wk is None) and (v_first is None) == (lam is None), "attn_prepare: arguments that come in pairs")
    for t in (v_keep, v_first):
        _need(t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.shape == (T, nkv * dv)), "attn_prepare: values float32 [T, nkv*dv]")
    _need(q_out.is_contiguous() and q_out.shape == (T, nh * maps * HD) and q_out.dtype == k_cache.dtype == v_cache.dtype
          and k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape[1] == nkv and v_cache.shape == k_cache.shape
          and HD >= max(maps * dk, dv), "attn_prepare: outputs")
    _need(positions.dtype == _I32 and positions.numel() >= T and (slot_mapping is None or (slot_mapping.dtype == _I32 and slot_mapping.numel() >= T)),
          "attn_prepare: positions / slot_mapping int32 [T]")
    _need(inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == rot), "attn_prepare: inv_freq float32 [rot/2]")
    fn = getattr(_lib(), "kvcm_attn_prepare_" + _suffix(q_out))
    _check(fn(_p(proj), proj.stride(0), _p(bias), _p(wq), _p(wk), _p(positions), _p(inv_freq), int(rot), int(bool(head_norm)),
              ctypes.c_float(eps), _p(v_keep), _p(v_first), _p(lam), _p(slot_mapping), B, _p(q_out), _p(k_cache), _p(v_cache),
              T, nh, nkv, dk, dv, HD, int(bool(interleaved)), _p(v_inv_freq), int(maps), _stream()), "attn_prepare", f"(nh={nh}, nkv={nkv}, dk={dk}, dv={dv}, HD={HD})")


# ------------------------------------------- blocks normalised on both sides, and what comes with them

def embed_scaled(ids: torch.Tensor, table: torch.Tensor, x: torch.Tensor, keep: Optional[torch.Tensor], scale: float) -> None:
    """x[t, :] = float(table[ids[t], :]) * scale; ``keep`` (optional, float32 like x) receives the same rows."""
    _cuda(ids, table, x, keep)
    T, H = x.shape
    _need(ids.dtype == _I32 and ids.numel() >= T and x.dtype == torch.float32 and x.is_contiguous() and table.is_contiguous()
          and table.shape[1] == H and (keep is None or (keep.dtype == torch.float32 and keep.is_contiguous() and keep.shape == x.shape)),
          "embed_scaled: layout")
    fn = getattr(_lib(), "kvcm_embed_scaled_" + _suffix(table))
    _check(fn(_p(ids), _p(table), _p(x), _p(keep), T, H, table.shape[0], ctypes.c_float(scale), _stream()), "embed_scaled")


def norm_post_pre(x: torch.Tensor, y: Optional[torch.Tensor], post_w: Optional[torch.Tensor], pre_w: Optional[torch.Tensor],
                  out: Optional[torch.Tensor], eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """The norm that closes a sublayer and the norm that opens the next one, in one pass over a row:
    x += post_w * y / rms(y) (when ``y`` is given; float32 like x), then out = pre_w * x / rms(x) (when ``out`` is
    given; storage dtype).  Weights are the multipliers themselves, float32 [H].  ``rows`` gathers: the norms are
    formed for rows[i] only, ``out`` has one row per index and x is left as it is."""
    _cuda(x, y, post_w, pre_w, out, rows)
    T, H = x.shape
    _need(x.dtype == torch.float32 and x.is_contiguous(), "norm_post_pre: x float32 [T, H]")
    _need(y is None or (y.dtype == torch.float32 and y.is_contiguous() and y.shape == x.shape and post_w is not None),
          "norm_post_pre: y float32 like x, with its weight")
    for w in (post_w, pre_w):
        _need(w is None or (w.dtype == torch.float32 and w.is_contiguous() and w.numel() == H), "norm_post_pre: weights float32 [H]")
    _need(out is not None or y is not None, "norm_post_pre: nothing to do")
    _need(out is None or (out.is_contiguous() and out.shape[1] == H and pre_w is not None), "norm_post_pre: out")
    n = T
    if rows is not None:
        _need(out is not None and rows.dtype == _I32 and rows.numel() >= out.shape[0], "norm_post_pre: rows int32 [n]")
        n = out.shape[0]
    elif out is not None:
        _need(out.shape[0] == T, "norm_post_pre: out rows != x rows")
    store = out.dtype if out is not None else torch.float32
    fn = getattr(_lib(), "kvcm_norm_post_pre_" + _SUFFIX[store])
    _check(fn(_p(x), _p(y), _p(post_w), _p(pre_w), _p(out), _p(rows), n, H, ctypes.c_float(eps), _stream()), "norm_post_pre",
           f"(hidden={H})")


def poly_norm_act(z: torch.Tensor, coef: torch.Tensor, out: torch.Tensor, eps: float) -> None:
    """out = a N(z) + b N(z^2) + c N(z^3) + e row by row, N(v) = v / sqrt(mean(v^2) + eps), powers element-wise;
    z float32 [T, F] (rows may be strided), coef float32 [4] = (a, b, c, e), out [T, F] in the storage dtype."""
    _cuda(z, coef, out)
    T, F = out.shape
    _need(z.dtype == torch.float32 and z.stride(1) == 1 and z.shape == out.shape and out.is_contiguous()
          and coef.dtype == torch.float32 and coef.is_contiguous() and coef.numel() == 4, "poly_norm_act: layout")
    fn = getattr(_lib(), "kvcm_poly_norm_act_" + _suffix(out))
    _check(fn(_p(z), z.stride(0), _p(coef), _p(out), T, F, ctypes.c_float(eps), _stream()), "poly_norm_act", f"(ff={F})")


def concat_cast(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = [a[t] | b[t]] in out's dtype; a, b float32 [T, H], out [T, 2H]."""
    _cuda(a, b, out)
    T, H = a.shape
    _need(a.dtype == b.dtype == torch.float32 and a.is_contiguous() and b.is_contiguous() and b.shape == a.shape
          and out.is_contiguous() and out.shape == (T, 2 * H), "concat_cast: layout")
    fn = getattr(_lib(), "kvcm_concat_cast_" + _suffix(out))
    _check(fn(_p(a), _p(b), _p(out), T, H, _stream()), "concat_cast")


def add_bias_rows(x: torch.Tensor, bias: torch.Tensor) -> None:
    """x[t, :] += bias, float32."""
    _cuda(x, bias)
    _need(x.dtype == bias.dtype == torch.float32 and x.is_contiguous() and bias.is_contiguous() and bias.numel() == x.shape[1],
          "add_bias_rows: layout")
    _check(_lib().kvcm_add_bias_rows(_p(x), _p(bias), x.shape[0], x.shape[1], _stream()), "add_bias_rows")


def softcap_rows(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap) in place, float32."""
    _cuda(x)
    _need(x.dtype == torch.float32 and x.is_contiguous(), "softcap_rows: float32")
    _check(_lib().kvcm_softcap_rows(_p(x), _ll(x.numel()), ctypes.c_float(cap), _stream()), "softcap_rows")


def rotate_heads(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, heads: int, head_dim: int,
                 interleaved: bool, sign: float = 1.0) -> None:
    """In place: the first 2 * len(inv_freq) elements of every head of row t turn by sign * positions[t] * inv_freq[i],
    pairs (2i, 2i+1) when ``interleaved`` else (i, i + n/2).  x [T, >= heads*head_dim] in either storage dtype;
    angles and the turn in float32."""
    _cuda(x, positions, inv_freq)
    T = x.shape[0]
    n = 2 * inv_freq.numel()
    _need(x.stride(1) == 1 and x.shape[1] >= heads * head_dim and inv_freq.dtype == torch.float32 and inv_freq.is_contiguous()
          and n <= head_dim and positions.dtype == _I32 and positions.numel() >= T, "rotate_heads: layout")
    fn = getattr(_lib(), "kvcm_rotate_heads_" + _suffix(x))
    _check(fn(_p(x), x.stride(0), _p(positions), _p(inv_freq), n, int(bool(interleaved)), ctypes.c_float(sign), T, heads,
              head_dim, _stream()), "rotate_heads")


def gla_prepare(qkv: torch.Tensor, q_base: int, n_q: int, qscale: float, z: torch.Tensor, bias: Optional[torch.Tensor],
                tau: float) -> None:
    """In place, float32: the n_q query elements of every row of ``qkv`` from ``q_base`` on are scaled by ``qscale``;
    ``z`` [T, heads*dk] becomes the decays sigmoid(z + bias)^(1/tau)."""
    _cuda(qkv, z, bias)
    T = qkv.shape[0]
    _need(qkv.dtype == z.dtype == torch.float32 and qkv.is_contiguous() and z.is_contiguous() and z.shape[0] == T
          and q_base + n_q <= qkv.shape[1] and (bias is None or (bias.dtype == torch.float32 and bias.is_contiguous()
                                                              and bias.numel() == z.shape[1])), "gla_prepare: layout")
    _check(_lib().kvcm_gla_prepare(_p(qkv), qkv.shape[1], int(q_base), int(n_q), ctypes.c_float(qscale), _p(z), _p(bias),
                                   z.shape[1], ctypes.c_float(tau), T, _stream()), "gla_prepare")


def latent_rope_cache(proj: torch.Tensor, wq: Optional[torch.Tensor], wc: torch.Tensor, positions: torch.Tensor,
                      inv_freq: torch.Tensor, interleaved: bool, slot_mapping: torch.Tensor, cq_out: Optional[torch.Tensor],
                      cache: torch.Tensor, q_rank: int, rank: int, rot_dim: int, eps: float) -> None:
    """Rows of ``proj`` (float32) are [dq: q_rank | c: rank | kr: rot_dim].  cq_out = wq * dq / rms(dq) (storage
    dtype; q_rank == 0: none); the row's page slot of ``cache`` [pages, 1, page, HD] becomes
    [wc * c / rms(c) | kr with its first 2 * len(inv_freq) elements turned by the position | zeros]."""
    _cuda(proj, wq, wc, positions, inv_freq, slot_mapping, cq_out, cache)
    T = proj.shape[0]
    HD = cache.shape[3]
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[1] >= q_rank + rank + rot_dim, "latent_rope_cache: proj")
    _need(cache.is_contiguous() and cache.shape[1] == 1 and HD >= rank + rot_dim, "latent_rope_cache: cache pages [pages, 1, page, HD]")
    _need(wc.dtype == torch.float32 and wc.numel() == rank and inv_freq.dtype == torch.float32 and 2 * inv_freq.numel() <= rot_dim,
          "latent_rope_cache: weights")
    if q_rank:
        _need(wq is not None and wq.dtype == torch.float32 and wq.numel() == q_rank and cq_out is not None and cq_out.is_contiguous()
              and cq_out.shape == (T, q_rank) and cq_out.dtype == cache.dtype, "latent_rope_cache: the query's latent")
    _need(positions.dtype == _I32 and slot_mapping.dtype == _I32 and positions.numel() >= T and slot_mapping.numel() >= T,
          "latent_rope_cache: positions / slot_mapping int32 [T]")
    fn = getattr(_lib(), "kvcm_latent_rope_cache_" + _suffix(cache))
    _check(fn(_p(proj), proj.stride(0), _p(wq), _p(wc), _p(positions), _p(inv_freq), 2 * inv_freq.numel(), int(bool(interleaved)),
              _p(slot_mapping), _p(cq_out), _p(cache), T, int(q_rank), int(rank), int(rot_dim), HD, ctypes.c_float(eps), _stream()),
           "latent_rope_cache")


def latent_q_rope(q: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, interleaved: bool, qn_out: torch.Tensor,
                  qrow: torch.Tensor, heads: int, dn: int, dr: int, rank: int) -> None:
    """Rows of ``q`` (float32) hold per head [unrotated: dn | rotated: dr].  qn_out [T, heads, dn] receives the
    unrotated parts in the storage dtype; qrow [T, heads, HD] receives at [rank : rank + dr] the rotated part turned by
    the position and zeros behind it ([0 : rank] is left for the map into the latent space)."""
    _cuda(q, positions, inv_freq, qn_out, qrow)
    T = q.shape[0]
    HD = qrow.shape[2]
    _need(q.dtype == torch.float32 and q.stride(1) == 1 and q.shape[1] >= heads * (dn + dr) and qn_out.is_contiguous()
          and qn_out.shape == (T, heads, dn) and qrow.is_contiguous() and qrow.shape[:2] == (T, heads) and HD >= rank + dr
          and qn_out.dtype == qrow.dtype and inv_freq.dtype == torch.float32 and 2 * inv_freq.numel() <= dr
          and positions.dtype == _I32 and positions.numel() >= T, "latent_q_rope: layout")
    fn = getattr(_lib(), "kvcm_latent_q_rope_" + _suffix(qrow))
    _check(fn(_p(q), q.stride(0), _p(positions), _p(inv_freq), 2 * inv_freq.numel(), int(bool(interleaved)), _p(qn_out), _p(qrow),
              T, heads, dn, dr, int(rank), HD, _stream()), "latent_q_rope")


# ------------------------------------------- several residual streams, differential and gated attention outputs

def embed_streams(ids: torch.Tensor, table: torch.Tensor, x: torch.Tensor) -> None:
    """x [T, S, D] float32: every one of the S residual streams of a row starts as the token's row of ``table``."""
    _cuda(ids, table, x)
    T, S, D = x.shape
    _need(x.dtype == torch.float32 and x.is_contiguous() and ids.dtype == _I32 and ids.numel() >= T and table.is_contiguous()
          and table.shape[1] == D, "embed_streams: x float32 [T, S, D], ids int32 [T], table [vocab, D]")
    fn = getattr(_lib(), "kvcm_embed_streams_" + _suffix(table))
    _check(fn(_p(ids), _p(table), _p(x), T, S, D, table.shape[0], _stream()), "embed_streams")


def hc_step(x: torch.Tensor, y: Optional[torch.Tensor], bias: Optional[torch.Tensor], mix: Optional[torch.Tensor],
            out_w: Optional[torch.Tensor], in_w: Optional[torch.Tensor], norm_w: Optional[torch.Tensor], h: Optional[torch.Tensor],
            eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """One pass over the residual streams x [T, S, D] (float32, in place).  With ``y`` (float32 [T, D], a sublayer's
    output; ``bias`` float32 [D] is added to it): x'_t = sum_s mix[s, t] x_s + out_w[t] y for all streams at once.
    With ``h`` ([n, D], storage dtype): u = sum_s in_w[s] x'_s and h = norm_w * u / sqrt(mean(u^2) + eps).  ``rows``
    gathers: only rows[i] are worked on and h has one row per index."""
    _cuda(x, y, bias, mix, out_w, in_w, norm_w, h, rows)
    T, S, D = x.shape
    _need(x.dtype == torch.float32 and x.is_contiguous(), "hc_step: x float32 [T, S, D]")
    _need(y is not None or h is not None, "hc_step: nothing to do")
    if y is not None:
        _need(y.dtype == torch.float32 and y.is_contiguous() and y.shape == (T, D) and mix is not None and out_w is not None
              and mix.dtype == out_w.dtype == torch.float32 and mix.is_contiguous() and mix.shape == (S, S) and out_w.numel() == S
              and (bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == D)),
              "hc_step: y float32 [T, D] with mix float32 [S, S], out float32 [S] (bias float32 [D])")
    n = T
    if h is not None:
        _need(in_w is not None and norm_w is not None and in_w.dtype == norm_w.dtype == torch.float32 and in_w.numel() == S
              and norm_w.is_contiguous() and norm_w.numel() == D and h.is_contiguous() and h.shape[1] == D,
              "hc_step: h [n, D] with in float32 [S] and the norm's weight float32 [D]")
    if rows is not None:
        _need(h is not None and rows.dtype == _I32 and rows.numel() >= h.shape[0], "hc_step: rows int32 [n]")
        n = h.shape[0]
    elif h is not None:
        _need(h.shape[0] == T, "hc_step: h rows != x rows")
    store = h.dtype if h is not None else torch.float32
    fn = getattr(_lib(), "kvcm_hc_step_" + _SUFFIX[store])
    _check(fn(_p(x), _p(y), _p(bias), _p(mix), _p(out_w), _p(in_w) if h is not None else None, _p(norm_w), _p(h), _p(rows), n, S, D,
              ctypes.c_float(eps), _stream()), "hc_step", f"(streams={S}, hidden={D})")


def diff_combine(a: torch.Tensor, gate: Optional[torch.Tensor], lam: torch.Tensor, out: torch.Tensor, heads: int, dv: int,
                 eps: float, post: float) -> None:
    """a [T, 2*heads, HD]: the attention outputs of the two maps of every head (heads 2h and 2h+1).  out [T, heads*dv] =
    (a1 - lam a2) / sqrt(mean_head((a1 - lam a2)^2) + eps) * post * sigmoid(gate[:, h]); ``gate`` float32 [T, >= heads]
    (a view with a row stride) or None; ``lam`` float32 [1] on the device."""
    _cuda(a, gate, lam, out)
    T, H2, HD = a.shape
    _need(a.is_contiguous() and H2 == 2 * heads and HD >= dv and out.is_contiguous() and out.shape == (T, heads * dv)
          and out.dtype == a.dtype and lam.dtype == torch.float32 and lam.numel() == 1, "diff_combine: layout")
    _need(gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[0] >= T and gate.shape[1] >= heads),
          "diff_combine: gate float32 [T, heads]")
    fn = getattr(_lib(), "kvcm_diff_combine_" + _suffix(a))
    _check(fn(_p(a), _p(gate), gate.stride(0) if gate is not None else 0, _p(lam), _p(out), T, heads, dv, HD, ctypes.c_float(eps),
              ctypes.c_float(post), _stream()), "diff_combine")


def gate_mul(x: torch.Tensor, gate: torch.Tensor, out: torch.Tensor) -> None:
    """out = x * sigmoid(gate), element by element; x and out [T, n] in the storage dtype, gate float32 [T, n] (row stride free)."""
    _cuda(x, gate, out)
    T, n = x.shape
    _need(x.is_contiguous() and out.is_contiguous() and out.shape == x.shape and out.dtype == x.dtype and gate.dtype == torch.float32
          and gate.stride(1) == 1 and gate.shape == (T, n), "gate_mul: layout")
    fn = getattr(_lib(), "kvcm_gate_mul_" + _suffix(x))
    _check(fn(_p(x), _p(gate), gate.stride(0), _p(out), T, n, _stream()), "gate_mul")
