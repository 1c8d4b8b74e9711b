"""Python face of the CUDA kernels: checks tensors, passes pointers and the
current stream to the ``extern "C"`` launchers, and raises on a refusal.

Nothing here computes on the host and nothing falls back: a CPU tensor or a
missing library is an error.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .csrc.build import load_library

IE_F32, IE_BF16 = 0, 1
_CODES = {torch.float32: IE_F32, torch.bfloat16: IE_BF16}
_ERRORS = {-1: "unsupported dtype combination", -2: "unsupported size", -3: "misaligned pointer or stride",
           -4: "size beyond the kernel's static limit"}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 and bfloat16, not {dtype}") from None


LAUNCHES = 0     # launchers called so far (graph replays add what their capture counted)

# Extra -D flags per library ("core", "stream", "tcgen05", "attn_tcgen05", "attn_mma"), read when a library is first
# loaded.  Empty in the product; a measurement or a test that wants a variant (clock notes, no programmatic
# dependent launch, a short spin limit) fills it before the first call or passes ``defines`` to the loader itself.
BUILD_DEFINES: dict[str, dict] = {}


def _check(status: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if status == 0:
        return
    if status < 0:
        raise KernelError(f"{what}: refused ({_ERRORS.get(status, status)})")
    raise KernelError(f"{what}: CUDA error {status} at launch")


def _ptr(t: torch.Tensor | None) -> int | None:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernels run on CUDA tensors only; there is no CPU path")
    return t.data_ptr()


def _stream() -> int:
    # the raw handle of the current stream of the current device, without building a Stream object: a step makes
    # a hundred launches, and the object cost more host time than everything else around a launch
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


_core = None


def core():
    global _core
    if _core is None:
        lib = load_library("core", defines=dict(BUILD_DEFINES.get("core", {})))
        P, I, F, L = c_void_p, c_int, c_float, c_longlong
        lib.ie_embed_gather.argtypes = [P, P, I, P, I, I, I, P]
        lib.ie_patch_tokens.argtypes = [P, P, P, I, P]
        lib.ie_patch_tokens.restype = c_int
        lib.ie_stamp.argtypes = [P, P]
        lib.ie_stamp.restype = c_int
        lib.ie_rmsnorm.argtypes = [P, P, P, I, P, I, P, I, I, F, P]
        lib.ie_residual_add.argtypes = [P, P, I, I, I, P]
        lib.ie_rope_kv_write.argtypes = [P, P, P, I, I, P, P, P, P, P, P, I, I, I, I, I, I, I, P]
        lib.ie_silu_mul.argtypes = [P, P, I, I, I, I, I, P]
        lib.ie_attention_general.argtypes = [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, P, I, P]
        lib.ie_gemm_simt.argtypes = [P, I, P, I, P, I, I, I, I, I, I, I, P]
        lib.ie_argmax.argtypes = [P, P, I, I, L, P]
        lib.ie_repetition_penalty.argtypes = [P, P, P, I, I, L, I, P]
        lib.ie_sample.argtypes = [P, P, P, I, I, L, P]
        for name in ("ie_embed_gather", "ie_rmsnorm", "ie_residual_add", "ie_rope_kv_write", "ie_silu_mul",
                     "ie_attention_general", "ie_gemm_simt", "ie_argmax", "ie_repetition_penalty", "ie_sample"):
            getattr(lib, name).restype = c_int
        _core = lib
        _apply_check_limits()
    return _core


# ------------------------------------------------------------------ elementwise
def embed_gather(ids: torch.Tensor, table: torch.Tensor, residual: torch.Tensor) -> None:
    """residual[n] = table[ids[n]] as float32."""
    assert ids.dtype == torch.int32 and residual.dtype == torch.float32 and table.is_contiguous()
    n, d = residual.shape
    _check(core().ie_embed_gather(_ptr(ids), _ptr(table), dtype_code(table.dtype), _ptr(residual), n, d,
                                  table.shape[0], _stream()), "embed_gather")


def patch_tokens(ids: torch.Tensor, src: torch.Tensor, prev: torch.Tensor) -> None:
    """ids[i] = prev[src[i]] where src[i] >= 0 (token ids that are still on the device)."""
    assert ids.dtype == src.dtype == prev.dtype == torch.int32 and src.shape[0] >= ids.shape[0]
    _check(core().ie_patch_tokens(_ptr(ids), _ptr(src), _ptr(prev), ids.shape[0], _stream()), "patch_tokens")


def stamp(slots: torch.Tensor, index: int) -> None:
    """slots[index] = the GPU's nanosecond clock once everything enqueued before has finished (int64 tensor);
    for timelines of a step.  Not counted as a launch of the step."""
    global LAUNCHES
    assert slots.dtype is torch.int64 and 0 <= index < slots.numel()
    _check(core().ie_stamp(slots.data_ptr() + 8 * index, _stream()), "stamp")
    LAUNCHES -= 1


def rmsnorm(residual: torch.Tensor, delta: torch.Tensor | None, gain: torch.Tensor, out: torch.Tensor,
            eps: float, row_index: torch.Tensor | None = None) -> None:
    """out = rmsnorm(residual (+ delta)) * gain; residual takes the sum unless rows are gathered."""
    d = residual.shape[-1]
    n_rows = out.shape[0]
    assert residual.dtype == torch.float32 and residual.is_contiguous() and out.is_contiguous()
    assert delta is None or (delta.dtype == out.dtype and delta.is_contiguous() and delta.shape == residual.shape)
    assert gain.shape == (d,) and out.shape[1] == d
    _check(core().ie_rmsnorm(_ptr(residual), _ptr(delta), _ptr(gain), dtype_code(gain.dtype), _ptr(out),
                             dtype_code(out.dtype), _ptr(row_index), n_rows, d, float(eps), _stream()), "rmsnorm")


def residual_add(residual: torch.Tensor, delta: torch.Tensor) -> None:
    n, d = residual.shape
    _check(core().ie_residual_add(_ptr(residual), _ptr(delta), dtype_code(delta.dtype), n, d, _stream()),
           "residual_add")


def rope_kv_write(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cos: torch.Tensor | None,
                  sin: torch.Tensor | None, positions: torch.Tensor, slot_mapping: torch.Tensor | None,
                  kpool: torch.Tensor | None, vpool: torch.Tensor | None, n_heads: int, n_kv_heads: int,
                  head_dim: int, page_size: int, rotate_q: bool = True) -> None:
    """Rotate q in place (unless ``rotate_q`` is off: the attention kernel then rotates it as it reads it);
    write rotated k and raw v into their page slots (if pools are given).

    q, k, v are row-strided views [n, heads*head_dim] (columns of one fused buffer, for instance).
    """
    n = q.shape[0]
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and k.stride(0) == v.stride(0)
    write = kpool is not None
    _check(core().ie_rope_kv_write(_ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0), _ptr(cos), _ptr(sin),
                                   _ptr(positions), _ptr(slot_mapping), _ptr(kpool), _ptr(vpool), n, n_heads,
                                   n_kv_heads, head_dim, page_size, (1 if write else 0) | (0 if rotate_q else 2),
                                   dtype_code(q.dtype),
                                   _stream()), "rope_kv_write")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """out[n, j] = silu(gate_j) * up_j; gate and up are the two halves of a row, or alternate when ``interleaved``."""
    n, inter = out.shape
    assert gate_up.shape == (n, 2 * inter) and gate_up.stride(1) == 1 and out.is_contiguous()
    _check(core().ie_silu_mul(_ptr(gate_up), _ptr(out), n, inter, gate_up.stride(0), 1 if interleaved else 0,
                              dtype_code(out.dtype), _stream()), "silu_mul")


# --------------------------------------------------------------------- attention
def attention_general(q: torch.Tensor, out: torch.Tensor, kpool: torch.Tensor, vpool: torch.Tensor,
                      block_table: torch.Tensor, q_start: torch.Tensor, ctx_before: torch.Tensor,
                      work_req: torch.Tensor, work_pair0: torch.Tensor, n_work: int, n_heads: int,
                      n_kv_heads: int, head_dim: int, page_size: int, window: int | None, scale: float,
                      score_bias: torch.Tensor | None = None) -> None:
    """Paged causal attention in float32 arithmetic.  ``score_bias`` (float32 [n_heads, D], contiguous) is added to
    the scaled score of a query at position p and a key at position j as ``score_bias[head, min(p - j, D - 1)]``."""
    assert q.stride(1) == 1 and out.stride(1) == 1 and kpool.dtype == q.dtype == out.dtype
    assert block_table.dtype == torch.int32 and block_table.stride(1) == 1
    if score_bias is not None:
        assert score_bias.dtype is torch.float32 and score_bias.is_contiguous() and score_bias.shape[0] == n_heads
    _check(core().ie_attention_general(_ptr(q), _ptr(out), _ptr(kpool), _ptr(vpool), _ptr(block_table),
                                       _ptr(q_start), _ptr(ctx_before), _ptr(work_req), _ptr(work_pair0),
                                       q.stride(0), out.stride(0), block_table.stride(0), n_work, n_heads,
                                       n_kv_heads, head_dim, page_size, int(window or 0), float(scale),
                                       dtype_code(q.dtype), _ptr(score_bias),
                                       score_bias.shape[1] if score_bias is not None else 0, _stream()),
           f"attention_general(head_dim={head_dim}, heads={n_heads}/{n_kv_heads})")


# -------------------------------------------------------------------------- gemm
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T in float32 arithmetic."""
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and out.shape == (m, n)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(core().ie_gemm_simt(_ptr(a), dtype_code(a.dtype), _ptr(w), dtype_code(w.dtype), _ptr(out),
                               dtype_code(out.dtype), m, n, k, a.stride(0), w.stride(0), out.stride(0),
                               _stream()), f"gemm_simt({a.dtype},{w.dtype}->{out.dtype})")


# ---------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    _check(core().ie_argmax(_ptr(logits), _ptr(out), logits.shape[0], logits.shape[1], logits.stride(0),
                            _stream()), "argmax")


def repetition_penalty(logits: torch.Tensor, context: torch.Tensor, penalty: torch.Tensor) -> None:
    assert logits.dtype == torch.float32 and context.dtype == torch.int32 and penalty.dtype == torch.float32
    assert context.is_contiguous() and context.shape[0] == logits.shape[0]
    _check(core().ie_repetition_penalty(_ptr(logits), _ptr(context), _ptr(penalty), logits.shape[0],
                                        logits.shape[1], logits.stride(0), context.shape[1], _stream()),
           "repetition_penalty")


def sample(logits: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """rows: int32 [n, 7] records (temperature bits, top_p bits, top_k, seed lo/hi, key lo/hi)."""
    assert logits.dtype == torch.float32 and rows.dtype == torch.int32 and rows.shape == (logits.shape[0], 7)
    assert rows.is_contiguous() and out.dtype == torch.int32
    _check(core().ie_sample(_ptr(logits), _ptr(rows), _ptr(out), logits.shape[0], logits.shape[1],
                            logits.stride(0), _stream()), "sample")


# ------------------------------------------------- tensor-core attention (bfloat16)
MMA_HEAD_DIMS = (64, 128)
_mma: dict[int, object] = {}


def attention_mma_library(head_dim: int):
    """The tensor-core attention kernels built for one head size; compiled when first asked for."""
    if head_dim not in MMA_HEAD_DIMS:
        raise KernelError(f"tensor-core attention is built for head sizes {MMA_HEAD_DIMS}, not {head_dim}")
    lib = _mma.get(head_dim)
    if lib is None:
        defines = {"IE_HD": head_dim, **BUILD_DEFINES.get("attn_mma", {})}
        lib = load_library(f"attn_mma_hd{head_dim}", ["attention_mma.cu"], defines, ["attention_noalloc.h"])
        P, I, F = c_void_p, c_int, c_float
        lib.ie_attention_prefill.argtypes = [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, P]
        lib.ie_attention_prefill.restype = c_int
        lib.ie_attention_decode.argtypes = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, I, P]
        lib.ie_attention_decode.restype = c_int
        lib.ie_attention_decode_fused.argtypes = [P] * 14 + [I] * 10 + [F, I, I, I, P]
        lib.ie_attention_decode_fused.restype = c_int
        lib.ie_attention_decode_scratch_floats.argtypes = [I, I, I]
        lib.ie_attention_decode_scratch_floats.restype = c_longlong
        lib.ie_attention_decode_ticket_words.restype = c_longlong
        lib.ie_attention_decode_warps.restype = c_int
        lib.ie_attention_decode_max_blocks.restype = c_int
        _mma[head_dim] = lib
        _apply_check_limits()
    return lib


def attention_prefill_mma(q, out, kpool, vpool, block_table, q_start, ctx_before, work_req, work_pair0, n_work,
                          n_heads, n_kv_heads, head_dim, page_size, window, scale, rows: int = 64) -> None:
    """Causal paged attention for any mix of portions and single tokens; bfloat16; the work list cuts each
    request's (token, head-in-group) pairs into tiles of ``rows`` (64 or 128)."""
    assert q.dtype is torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    lib = attention_mma_library(head_dim)
    _check(lib.ie_attention_prefill(_ptr(q), _ptr(out), _ptr(kpool), _ptr(vpool), _ptr(block_table), _ptr(q_start),
                                    _ptr(ctx_before), _ptr(work_req), _ptr(work_pair0), q.stride(0), out.stride(0),
                                    block_table.stride(0), n_work, n_heads, n_kv_heads, head_dim, page_size,
                                    int(window or 0), float(scale), rows, _stream()), "attention_prefill_mma")


def attention_decode_scratch_floats(n_tokens, n_heads, n_splits, head_dim) -> int:
    return int(attention_mma_library(head_dim).ie_attention_decode_scratch_floats(n_tokens, n_heads, n_splits))


def attention_decode_geometry(head_dim) -> tuple[int, int]:
    """(warps, i.e. splits, of a decode block; the most blocks per (request, kv head) a launch takes)."""
    lib = attention_mma_library(head_dim)
    return int(lib.ie_attention_decode_warps()), int(lib.ie_attention_decode_max_blocks())


def attention_decode_ticket_words(head_dim) -> int:
    """How many words at the start of the decode scratch hold tickets; they must be zero before the
    first launch on a piece of scratch (every launch leaves them zero)."""
    return int(attention_mma_library(head_dim).ie_attention_decode_ticket_words())


def attention_decode_mma(q, out, kpool, vpool, block_table, q_start, ctx_before, scratch, n_requests, n_tokens,
                         n_heads, n_kv_heads, head_dim, page_size, window, scale, n_splits, split_keys) -> None:
    """Split-key attention for steps where every request brings at most 16 (token, head-in-group) rows.

    ``scratch`` is float32 device memory of ``attention_decode_scratch_floats`` elements: partial
    tickets in its first ``attention_decode_ticket_words`` words, which must be zero when the first
    launch starts and are zero again when a launch ends, then partial outputs, maxima and sums of
    every block, which are written before they are read.  At most warps x blocks of
    ``attention_decode_geometry`` splits, each a multiple of 32 keys."""
    assert q.dtype is torch.bfloat16 and scratch.dtype is torch.float32
    lib = attention_mma_library(head_dim)
    _check(lib.ie_attention_decode(_ptr(q), _ptr(out), _ptr(kpool), _ptr(vpool), _ptr(block_table), _ptr(q_start),
                                   _ptr(ctx_before), _ptr(scratch), q.stride(0), out.stride(0),
                                   block_table.stride(0), n_requests, n_tokens, n_heads, n_kv_heads, head_dim,
                                   page_size, int(window or 0), float(scale), n_splits, split_keys, _stream()),
           "attention_decode_mma")


def attention_decode_fused(q, k_new, v_new, out, kpool, vpool, block_table, q_start, ctx_before, scratch, cos, sin,
                           positions, slot_mapping, n_requests, n_heads, n_kv_heads, head_dim, page_size, window,
                           scale, write_kv, n_splits, split_keys) -> None:
    """``attention_decode_mma`` for steps in which every request brings exactly one token, with the rotary
    encoding and the cache write folded in: ``q`` and ``k_new`` arrive unrotated; with ``write_kv`` the
    token's key (rotated) and value join the keys of the step and are stored at ``slot_mapping`` in the
    pools.  ``cos``/``sin`` are float32 tables [positions, head_dim/2], or None for no rotation."""
    assert q.dtype is torch.bfloat16 and scratch.dtype is torch.float32
    assert k_new.stride(0) == v_new.stride(0) and k_new.stride(1) == 1 and v_new.stride(1) == 1
    lib = attention_mma_library(head_dim)
    _check(lib.ie_attention_decode_fused(_ptr(q), _ptr(k_new), _ptr(v_new), _ptr(out), _ptr(kpool), _ptr(vpool),
                                         _ptr(block_table), _ptr(q_start), _ptr(ctx_before), _ptr(scratch),
                                         _ptr(cos), _ptr(sin), _ptr(positions), _ptr(slot_mapping), q.stride(0),
                                         k_new.stride(0), out.stride(0), block_table.stride(0), n_requests, n_heads,
                                         n_kv_heads, head_dim, page_size, int(window or 0), float(scale),
                                         1 if write_kv else 0, n_splits, split_keys, _stream()),
           "attention_decode_fused")


# ----------------------------------------------- weight-streaming product for few rows
STREAM_MAX_ROWS = 64        # what the kernel takes
STREAM_BEST_ROWS = 16       # beyond this the library product is faster (activations are re-read per block)
_EPI = {"bf16": 0, "f32": 1, "residual": 2, "silu_mul": 3, "residual_normout": 4}
SSQ_SLOT = 16               # rows of a sums-of-squares array ([SSQ_SLOT, blocks]: a block's sum for each activation row)
_stream_lib = None
_stream_variants: dict = {}


def _bind_stream(lib):
    P, I, F = c_void_p, c_int, c_float
    lib.ie_gemm_stream.argtypes = [P, P, P, P, I, P, I, I, I, I, I, I, F, I, I, I, P]
    lib.ie_gemm_stream.restype = c_int
    lib.ie_gemm_stream_tma.argtypes = [P, P, P, P, I, P, I, I, I, I, I, I, F, I, I, I, P, I, P, I, P, I, P]
    lib.ie_gemm_stream_tma.restype = c_int
    lib.ie_gemm_stream_tma_supports.argtypes = [I, I, I, I]
    lib.ie_gemm_stream_tma_supports.restype = c_int
    lib.ie_gemm_stream_tma_error.restype = c_int
    return lib


def stream_library(defines: dict | None = None):
    """The streaming products' library.  With ``defines`` a variant compiled with those -D flags (kept apart from the
    product's own; ``gemm_stream(..., lib=...)`` runs it)."""
    global _stream_lib
    if defines:
        key = repr(sorted(defines.items()))
        if key not in _stream_variants:
            _stream_variants[key] = _bind_stream(load_library("stream", ["gemm_stream.cu", "gemm_stream_tma.cu"], dict(defines)))
        return _stream_variants[key]
    if _stream_lib is None:
        _stream_lib = _bind_stream(load_library("stream", ["gemm_stream.cu", "gemm_stream_tma.cu"],
                                                dict(BUILD_DEFINES.get("stream", {}))))
    return _stream_lib


_n_sms: dict[int, int] = {}


def sm_count() -> int:
    dev = torch.cuda.current_device()
    if dev not in _n_sms:
        _n_sms[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _n_sms[dev]


def stream_error(lib=None) -> int:
    """Reads and clears the error word of the bulk-copy streaming kernel (0: no wait ever timed out)."""
    return int((lib or stream_library()).ie_gemm_stream_tma_error())


def gemm_stream_ring_supports(m: int, n: int, k: int, normed: bool) -> bool:
    """Whether the streaming kernel with the shared-memory ring takes m rows of k columns (with a norm in its
    prologue: the rows must then fit in shared memory beside the ring)."""
    return bool(stream_library().ie_gemm_stream_tma_supports(m, n, k, 1 if normed else 0))


def gemm_stream(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, m: int, epi: str = "bf16",
                gain: torch.Tensor | None = None, eps: float = 0.0, row_index: torch.Tensor | None = None,
                nt: int | None = None, prenormed=None, normout=None, lib=None) -> None:
    """c = a @ w^T for m <= 64 rows, bfloat16 weights, reading w once at HBM speed.

    With ``gain`` the input ``a`` is the float32 residual stream (rows gathered by ``row_index`` if given)
    and RMSNorm with that gain and ``eps`` is applied inside the kernel.  ``epi``: "bf16" or "f32" store,
    "residual" adds into the float32 ``c``, "silu_mul" takes w's rows as alternating gate/up and writes
    silu(gate)*up, half as wide.

    Two products can hand a norm over between them.  ``normout=(xg, gain_next, ssq)`` with epi "residual":
    besides adding into ``c`` the kernel writes ``xg`` = bfloat16(new c * gain_next) and, per block, the sums of
    squares of the new rows into ``ssq`` ([SSQ_SLOT rows, SMs] float32).  ``prenormed=(xg, ssq)`` with ``eps``: ``a`` is
    ignored, the input is ``xg`` and the 1/rms comes from ``ssq``: RMSNorm without reading the residual again."""
    n, k = w.shape
    assert w.dtype is torch.bfloat16 and w.stride(1) == 1 and a.stride(-1) == 1 and c.stride(-1) == 1
    lib = lib or stream_library()
    if prenormed is not None or normout is not None:
        pro = 2 if prenormed is not None else 0
        xg, ssq = (prenormed if prenormed is not None else (normout[0], normout[2]))
        gain_next = normout[1] if normout is not None else None
        src = xg if prenormed is not None else a
        assert src.dtype is torch.bfloat16 and xg.dtype is torch.bfloat16 and ssq.dtype is torch.float32
        assert nt is None and lib.ie_gemm_stream_tma_supports(m, n, k, pro)
        code = _EPI["residual_normout"] if normout is not None else _EPI[epi]
        _check(lib.ie_gemm_stream_tma(_ptr(src), _ptr(w), _ptr(c), None, 0, None, m, n, k, src.stride(0), w.stride(0),
                                      c.stride(0), float(eps), pro, code, sm_count(), _ptr(xg), xg.stride(0),
                                      _ptr(gain_next), dtype_code(gain_next.dtype) if gain_next is not None else 0,
                                      _ptr(ssq), ssq.shape[1], _stream()),
               f"gemm_stream_tma(m={m}, n={n}, k={k}, {epi}, handed-over norm)")
        return
    if gain is None:
        assert a.dtype is torch.bfloat16
    else:
        assert a.dtype is torch.float32 and gain.shape == (k,)
    if nt is None and lib.ie_gemm_stream_tma_supports(m, n, k, 0 if gain is None else 1):
        # persistent bulk-copy kernel: one block per SM, weights through a ring of shared memory
        _check(lib.ie_gemm_stream_tma(_ptr(a), _ptr(w), _ptr(c), _ptr(gain),
                                      dtype_code(gain.dtype) if gain is not None else 0, _ptr(row_index), m, n, k,
                                      a.stride(0), w.stride(0), c.stride(0), float(eps),
                                      0 if gain is None else 1, _EPI[epi], sm_count(), None, 0, None, 0, None, 0,
                                      _stream()),
               f"gemm_stream_tma(m={m}, n={n}, k={k}, {epi})")
        return
    if nt is None:
        nt = 4 if n >= 16384 else (2 if n >= 8192 else 1)
        if m > 32:
            nt = min(nt, 2)
    _check(lib.ie_gemm_stream(_ptr(a), _ptr(w), _ptr(c), _ptr(gain),
                                           dtype_code(gain.dtype) if gain is not None else 0, _ptr(row_index), m, n, k,
                                           a.stride(0), w.stride(0), c.stride(0), float(eps),
                                           0 if gain is None else 1, _EPI[epi], nt, _stream()),
           f"gemm_stream(m={m}, n={n}, k={k}, {epi})")


# ------------------------------------------------ tcgen05 product for many rows (prompt portions)
_tc_lib = None


def tcgen05_library():
    global _tc_lib
    if _tc_lib is None:
        lib = load_library("tcgen05", ["gemm_tcgen05.cu"], dict(BUILD_DEFINES.get("tcgen05", {})))
        P, I = c_void_p, c_int
        lib.ie_gemm_tcgen05.argtypes = [P, P, P, I, I, I, I, I, I, I, I, I, P]
        lib.ie_gemm_tcgen05.restype = c_int
        lib.ie_gemm_tcgen05_supports.argtypes = [I, I, I, I, I]
        lib.ie_gemm_tcgen05_supports.restype = c_int
        lib.ie_gemm_tcgen05_error.restype = c_int
        _tc_lib = lib
    return _tc_lib


def gemm_tcgen05_supports(m: int, n: int, k: int, lda: int, ldw: int) -> bool:
    return bool(tcgen05_library().ie_gemm_tcgen05_supports(m, n, k, lda, ldw))


def gemm_tcgen05_error() -> int:
    """Reads and clears the error word that a timed-out wait of the tcgen05 kernel leaves (0: none)."""
    return int(tcgen05_library().ie_gemm_tcgen05_error())


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epi: str = "bf16", bn: int = 256) -> None:
    """c = a @ w^T on the fifth-generation tensor cores (TMA operands, accumulator in tensor memory).

    ``epi``: "bf16" store, "residual" adds into the float32 ``c``, "silu_mul" takes w's rows as alternating
    gate/up and writes silu(gate)*up, half as wide.  ``bn``: tile width, 128 or 256."""
    m, k = a.shape
    n = w.shape[0]
    assert a.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and a.stride(1) == 1 and w.stride(1) == 1
    _check(tcgen05_library().ie_gemm_tcgen05(_ptr(a), _ptr(w), _ptr(c), m, n, k, a.stride(0), w.stride(0), c.stride(0),
                                             _EPI[epi], bn, sm_count(), _stream()), f"gemm_tcgen05(m={m}, n={n}, k={k}, {epi})")


# ------------------------------------------- prompt-portion attention on tcgen05 (head sizes 64 and 128)
_fa5_lib = None


def attention_tcgen05_library():
    global _fa5_lib
    if _fa5_lib is None:
        lib = load_library("attn_tcgen05", ["attention_tcgen05.cu"], dict(BUILD_DEFINES.get("attn_tcgen05", {})))
        P, I = c_void_p, c_int
        lib.ie_attention_tcgen05.argtypes = [P] * 9 + [I] * 9 + [c_float, P, P, P, P]
        lib.ie_attention_tcgen05.restype = c_int
        lib.ie_attention_tcgen05_supports.argtypes = [I, I, I]
        lib.ie_attention_tcgen05_supports.restype = c_int
        lib.ie_attention_tcgen05_error.restype = c_int
        _fa5_lib = lib
        _apply_check_limits()
    return _fa5_lib


def attention_tcgen05_supports(head_dim: int, page_size: int, window) -> bool:
    return bool(attention_tcgen05_library().ie_attention_tcgen05_supports(head_dim, page_size, int(window or 0)))


def attention_tcgen05_error() -> int:
    """Reads and clears the error word that a timed-out wait of the kernel leaves (0: none)."""
    return int(attention_tcgen05_library().ie_attention_tcgen05_error())


def attention_tcgen05(q, out, kpool, vpool, block_table, q_start, ctx_before, work_req, work_pair0, n_work,
                      n_heads, n_kv_heads, head_dim, page_size, scale, cos=None, sin=None, positions=None) -> None:
    """Causal paged attention for prompt portions with tcgen05 tensor cores; bfloat16, head size 64 or 128;
    the work list cuts each request's (token, head-in-group) rows into tiles of 128.  ``kpool``/``vpool``
    are one layer's pages, [pages, kv_heads, page_size, head_dim], contiguous.  With ``cos``/``sin`` (float32
    [positions, head_dim/2]) and ``positions`` (int32 per token) q arrives unrotated and is rotated as read."""
    assert q.dtype is torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert kpool.is_contiguous() and vpool.is_contiguous() and kpool.dim() == 4
    _check(attention_tcgen05_library().ie_attention_tcgen05(
        _ptr(q), _ptr(out), _ptr(kpool), _ptr(vpool), _ptr(block_table), _ptr(q_start), _ptr(ctx_before),
        _ptr(work_req), _ptr(work_pair0), q.stride(0), out.stride(0), block_table.stride(0), n_work, n_heads,
        n_kv_heads, head_dim, page_size, kpool.shape[0], float(scale), _ptr(cos), _ptr(sin), _ptr(positions),
        _stream()), "attention_tcgen05")


# ------------------------------------------------ a checks build: page ids, slots and token ids compared with limits
# (the device has no sanitizer here: this is what stands in for one while debugging a cache manager or a new part)
CHECK_LIBRARIES = ("core", "attn_mma", "attn_tcgen05")
CHECK_UNITS = ("elementwise", "attention_general", "attention_mma", "attention_tcgen05")
CHECK_CODES = {1: "page id", 2: "cache slot", 3: "token id"}
_check_limits: tuple[int, int, int] | None = None


def enable_checks() -> None:
    """Build the kernels that read page ids, cache slots and token ids from memory with ``-DIE_CHECKS=1``: a value out
    of range is recorded and replaced by a safe one instead of being used.  Call before the first kernel runs (a
    library that is already loaded stays as it was built); then ``set_check_limits``, and ``check_device_errors`` or
    ``read_check_words`` after the steps in question."""
    for name in CHECK_LIBRARIES:
        BUILD_DEFINES.setdefault(name, {})["IE_CHECKS"] = 1


def checks_enabled() -> bool:
    return any(BUILD_DEFINES.get(name, {}).get("IE_CHECKS") for name in CHECK_LIBRARIES)


def _loaded_check_functions(prefix: str):
    from .csrc import build as _build
    for lib in list(_build._loaded.values()):
        for unit in CHECK_UNITS:
            try:
                fn = getattr(lib, f"{prefix}_{unit}")
            except AttributeError:
                continue
            yield unit, fn


def _apply_check_limits() -> None:
    if _check_limits is None:
        return
    for unit, fn in _loaded_check_functions("ie_check_limits"):
        fn.argtypes = [c_int, c_int, c_int]
        fn.restype = c_int
        _check(fn(*_check_limits), f"ie_check_limits_{unit}")


def set_check_limits(n_pages: int, n_slots: int, vocab: int) -> None:
    """The limits of a checks build: page ids below ``n_pages``, cache slots below ``n_slots``, token ids below
    ``vocab`` (libraries that load later get them when they load)."""
    global _check_limits
    _check_limits = (int(n_pages), int(n_slots), int(vocab))
    _apply_check_limits()


def read_check_words() -> list[tuple[str, str, int, int, int]]:
    """(unit, what, first bad value, its limit, how many) for every unit of a checks build that saw a value out of
    range since the last call; synchronises the device."""
    import ctypes
    out = []
    for unit, fn in _loaded_check_functions("ie_check_read"):
        word = (ctypes.c_int * 4)()
        fn.argtypes = [c_void_p]
        fn.restype = c_int
        _check(fn(ctypes.addressof(word)), f"ie_check_read_{unit}")
        if word[3]:
            out.append((unit, CHECK_CODES.get(word[0], str(word[0])), int(word[1]), int(word[2]), int(word[3])))
    return out


def check_device_errors() -> None:
    """Reads the error words of the kernels that wait on barriers (a wait that ran out records a code and the
    kernel leaves early) and raises if any is set.  It synchronises the device, so it belongs where the
    engine is idle anyway: after a replayed step, at the end of a generation."""
    found = []
    if _stream_lib is not None and (e := stream_error()):
        found.append(f"streaming product: code {e}")
    if _tc_lib is not None and (e := gemm_tcgen05_error()):
        found.append(f"tcgen05 product: code {e}")
    if _fa5_lib is not None and (e := attention_tcgen05_error()):
        found.append(f"tcgen05 attention: code {e}")
    if found:
        raise KernelError("a kernel gave up a bounded wait; its results are not valid (" + "; ".join(found) + ")")
    if checks_enabled():
        bad = read_check_words()
        if bad:
            raise KernelError("checks build: " + "; ".join(
                f"{unit} read {n} value(s) out of range, the first a {what} of {v} (limit {lim})" for unit, what, v, lim, n in bad))
