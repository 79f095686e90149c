"""Python wrappers of the hand-written CUDA kernels.

Every wrapper checks device, dtype, shape and contiguity, then launches on the
current CUDA stream through the compiled library's C entry point.  There is no
CPU or library fallback: a tensor that is not on a CUDA device, or a library
that cannot be built, raises.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..csrc.build import ExtensionError, load_library

DT_CODE = {torch.float32: 0, torch.bfloat16: 1}

# number of this package's kernels launched since import (a graph replay adds its node count)
launch_count = 0
DECODE_TMA_CLUSTER_SPLITS = 16  # CLUSTER_SPLITS_MAX of csrc/attention_tc.cu


class KernelError(RuntimeError):
    pass


_ERRORS = {1001: "size or option not supported by this kernel"}


def _check(code: int, what: str) -> None:
    global launch_count
    if code != 0:
        detail = _ERRORS.get(code)
        if detail is None:
            try:
                detail = torch.cuda.cudart().cudaGetErrorString(code)  # type: ignore[attr-defined]
            except Exception:
                detail = f"CUDA error {code}"
        raise KernelError(f"{what}: {detail} (code {code})")
    launch_count += 1


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _sink(sink) -> float:
    """The attention kernels' sink argument: the score of one more term of the softmax denominator that has no
    value (exp(sink) is added to the sum of the exponentials), or -inf for none (also when a tensor gives a score per
    query head: ``_sink_heads``)."""
    return float("-inf") if sink is None or isinstance(sink, torch.Tensor) else float(sink)


def _sink_heads(sink, num_heads: int) -> c_void_p:
    """The attention kernels' second sink argument: a float32 score per query head (a learned sink), or null."""
    if not isinstance(sink, torch.Tensor):
        return c_void_p(0)
    _need(sink, "sink", torch.float32)
    if sink.numel() != num_heads:
        raise KernelError("a sink per head needs one score for every query head")
    return _ptr(sink)


def _need(t: torch.Tensor, name: str, dtype: torch.dtype | None = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor: the engine has no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, is {t.dtype}")


_fns: dict[str, ctypes._CFuncPtr] = {}


def _fn(source: str, name: str, argtypes: list, defines: dict | None = None):
    key = f"{source}:{name}:{sorted((defines or {}).items())}"
    f = _fns.get(key)
    if f is None:
        lib = load_library(source, defines)
        try:
            f = getattr(lib, name)
        except AttributeError as exc:
            raise ExtensionError(f"{name} missing from {source}") from exc
        f.argtypes = argtypes
        f.restype = c_int
        _fns[key] = f
    return f


# ------------------------------------------------------------------ elementwise


def embedding(h: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> None:
    """h[t] = float32(table[ids[t]]); h is the float32 residual stream [n, H]."""
    _need(h, "h", torch.float32), _need(table, "table"), _need(ids, "ids", torch.int32)
    n, H = h.shape
    if table.shape[1] != H or ids.numel() != n or table.dtype not in DT_CODE:
        raise KernelError("embedding: shapes or dtype do not agree")
    f = _fn("elementwise.cu", "dli_embedding", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(h), _ptr(table), _ptr(ids), n, H, DT_CODE[table.dtype], _stream()), "embedding")


def patch_tokens(ids: torch.Tensor, source: torch.Tensor, src: torch.Tensor) -> None:
    """ids[i] = source[src[i]] wherever src[i] >= 0: the token ids of a step that were sampled on
    the device by the step before and have not been read by the host."""
    _need(ids, "ids", torch.int32), _need(source, "source", torch.int32), _need(src, "src", torch.int32)
    if src.numel() != ids.numel():
        raise KernelError("patch_tokens: one source row per token")
    f = _fn("elementwise.cu", "dli_patch_tokens", [c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(ids), _ptr(source), _ptr(src), ids.numel(), _stream()), "patch_tokens")


def copy_page(pool: torch.Tensor, src: int, dst: int) -> None:
    """pool[:, dst] = pool[:, src] for a cache pool [layers, pages, ...] (copy-on-write of a forked
    request's last page)."""
    _need(pool, "pool")
    if pool.dim() < 2 or not (0 <= src < pool.shape[1] and 0 <= dst < pool.shape[1]):
        raise KernelError("copy_page: pool must be [layers, pages, ...] and the pages inside it")
    page_bytes = pool[0, 0].numel() * pool.element_size()
    f = _fn("elementwise.cu", "dli_copy_page", [c_void_p, c_longlong, c_longlong, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(pool), pool.shape[1] * page_bytes, page_bytes, pool.shape[0], src, dst, _stream()), "copy_page")


def add_rmsnorm(
    y: torch.Tensor,
    h: torch.Tensor,
    delta: torch.Tensor | None,
    weight: torch.Tensor,
    eps: float,
    rows: torch.Tensor | None = None,
) -> None:
    """y[r] = rmsnorm(h[s] + delta[s]) * weight with s = rows[r] (or r).

    Without ``rows`` the sum is written back to ``h`` (the residual stream moves on);
    with ``rows`` only the selected rows are read and ``h`` is left alone.
    """
    _need(y, "y"), _need(h, "h", torch.float32), _need(weight, "weight", torch.float32)
    H = h.shape[1]
    n_rows = y.shape[0]
    if y.dtype not in DT_CODE or y.shape[1] != H or weight.numel() != H:
        raise KernelError("add_rmsnorm: shapes or dtype do not agree")
    if delta is not None:
        _need(delta, "delta", y.dtype)
        if delta.shape != h.shape:
            raise KernelError("add_rmsnorm: delta and h differ in shape")
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() != n_rows:
            raise KernelError("add_rmsnorm: one output row per entry of rows")
    elif n_rows != h.shape[0]:
        raise KernelError("add_rmsnorm: y and h differ in rows")
    f = _fn(
        "elementwise.cu", "dli_add_rmsnorm",
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
    )
    _check(f(_ptr(y), _ptr(h), _ptr(delta), _ptr(weight), _ptr(rows), n_rows, H, eps, DT_CODE[y.dtype], _stream()), "add_rmsnorm")


def rotary_store(
    qkv: torch.Tensor,
    positions: torch.Tensor,
    inv_freq: torch.Tensor | None,
    slots: torch.Tensor | None,
    k_pool: torch.Tensor | None,
    v_pool: torch.Tensor | None,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    rotary_dim: int,
    page_size: int,
    write_kv: bool = True,
    table: torch.Tensor | None = None,
) -> None:
    """Rotate q and k heads of qkv [n, (nh + 2 nkv) d] by position; q in place, k and v into
    one layer's pools [pages, nkv, page_size, d] at ``slots`` (page * page_size + offset).
    ``table`` [n, rotary_dim] (from rotary_table) spares the kernel the sines and cosines."""
    _need(qkv, "qkv"), _need(positions, "positions", torch.int32)
    n = qkv.shape[0]
    if qkv.dtype not in DT_CODE or qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim or positions.numel() != n:
        raise KernelError("rotary_store: shapes or dtype do not agree")
    if rotary_dim:
        if inv_freq is None:
            raise KernelError("rotary_store: inv_freq is needed when rotary_dim > 0")
        _need(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("rotary_store: inv_freq must have rotary_dim / 2 entries")
    if write_kv:
        if slots is None or k_pool is None or v_pool is None:
            raise KernelError("rotary_store: slots and pools are needed to write keys and values")
        _need(slots, "slots", torch.int32), _need(k_pool, "k_pool", qkv.dtype), _need(v_pool, "v_pool", qkv.dtype)
        if tuple(k_pool.shape[1:]) != (num_kv_heads, page_size, head_dim) or k_pool.shape != v_pool.shape or slots.numel() != n:
            raise KernelError("rotary_store: pool layout must be [pages, kv_heads, page_size, head_dim]")
    if table is not None:
        _need(table, "table", torch.float32)
        if tuple(table.shape) != (n, rotary_dim):
            raise KernelError("rotary_store: table must be [n, rotary_dim]")
    f = _fn(
        "elementwise.cu", "dli_rotary_store",
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 8 + [c_void_p],
    )
    _check(
        f(_ptr(qkv), _ptr(positions), _ptr(inv_freq), _ptr(table), _ptr(slots), _ptr(k_pool), _ptr(v_pool), n, num_heads, num_kv_heads,
          head_dim, rotary_dim, page_size, int(write_kv), DT_CODE[qkv.dtype], _stream()),
        "rotary_store",
    )


def rotary_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """cos | sin of float32(position) * inv_freq for every token: float32 [n, 2 * len(inv_freq)]."""
    _need(positions, "positions", torch.int32), _need(inv_freq, "inv_freq", torch.float32)
    n, rot = positions.numel(), 2 * inv_freq.numel()
    table = torch.empty((n, rot), dtype=torch.float32, device=positions.device)
    f = _fn("elementwise.cu", "dli_rotary_table", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(table), _ptr(positions), _ptr(inv_freq), n, rot, _stream()), "rotary_table")
    return table


# what a gated feed-forward may apply to its gate; quick_gelu(g) = g * sigmoid(1.702 g)
GLU_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "quick_gelu": 2}


def silu_mul(out: torch.Tensor, gate_up: torch.Tensor, tiled: bool = False, activation: str = "silu", limit: float = 0.0,
             up_shift: float = 0.0) -> None:
    """out[n, I] = act(gate) * (up + up_shift), act = silu or another of GLU_ACTIVATIONS; with ``limit`` > 0 the gate is
    bounded from above by it and up to [-limit, limit] first.  gate_up [n, 2 I] holds gate | up side by
    side, or, ``tiled`` (I a multiple of 64), blocks of 128 columns: 64 gate features, then the same 64 up features."""
    _need(out, "out"), _need(gate_up, "gate_up", out.dtype)
    n, I = out.shape
    if out.dtype not in DT_CODE or tuple(gate_up.shape) != (n, 2 * I) or (tiled and I % 64) or activation not in GLU_ACTIVATIONS:
        raise KernelError("silu_mul: shapes, dtype or activation do not agree")
    f = _fn("elementwise.cu", "dli_silu_mul", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(gate_up), n, I, int(tiled), GLU_ACTIVATIONS[activation], float(limit), float(up_shift), DT_CODE[out.dtype],
             _stream()), "silu_mul")


def add_rmsnorm_pair(y1: torch.Tensor, y2: torch.Tensor | None, h: torch.Tensor, a: torch.Tensor | None, b: torch.Tensor | None,
                     w1: torch.Tensor, w2: torch.Tensor | None, eps: float, rows: torch.Tensor | None = None) -> None:
    """v = h[s] + (a[s] + b[s]) (either may be None), y1[r] = v / rms(v) * w1 and, if ``y2``, y2[r] = v / rms(v) * w2,
    with s = rows[r] (or r): two norms of one stream that differ in their weights only share the sum of squares.
    Without ``rows`` v is written back to ``h``.  All arithmetic float32."""
    _need(y1, "y1"), _need(h, "h", torch.float32), _need(w1, "w1", torch.float32)
    H = h.shape[1]
    n_rows = y1.shape[0]
    if y1.dtype not in DT_CODE or y1.shape[1] != H or w1.numel() != H:
        raise KernelError("add_rmsnorm_pair: shapes or dtype do not agree")
    if (y2 is None) != (w2 is None):
        raise KernelError("add_rmsnorm_pair: a second output needs a second weight")
    if y2 is not None:
        _need(y2, "y2", y1.dtype), _need(w2, "w2", torch.float32)
        if y2.shape != y1.shape or w2.numel() != H:
            raise KernelError("add_rmsnorm_pair: y2 and w2 must match y1 and w1")
    for d, name in ((a, "a"), (b, "b")):
        if d is not None:
            _need(d, name, y1.dtype)
            if d.shape != h.shape:
                raise KernelError(f"add_rmsnorm_pair: {name} and h differ in shape")
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() != n_rows:
            raise KernelError("add_rmsnorm_pair: one output row per entry of rows")
    elif n_rows != h.shape[0]:
        raise KernelError("add_rmsnorm_pair: y1 and h differ in rows")
    f = _fn("elementwise.cu", "dli_add_rmsnorm_pair",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    _check(f(_ptr(y1), _ptr(y2), _ptr(h), _ptr(a), _ptr(b), _ptr(w1), _ptr(w2), _ptr(rows), n_rows, H, eps, DT_CODE[y1.dtype], _stream()),
           "add_rmsnorm_pair")


def scale_softcap(logits: torch.Tensor, scale: float, cap: float) -> None:
    """logits <- logits * scale, then, if cap > 0, cap * tanh(logits / cap); float32, in place."""
    _need(logits, "logits", torch.float32)
    f = _fn("elementwise.cu", "dli_scale_softcap", [c_void_p, c_longlong, c_float, c_float, c_void_p])
    _check(f(_ptr(logits), logits.numel(), scale, cap, _stream()), "scale_softcap")


# ------------------------------------------------------------------ attention


SIMT_MAX_HEAD_DIM = 1024


def paged_attention_simt(
    out: torch.Tensor,
    qkv: torch.Tensor,
    k_pool: torch.Tensor,
    v_pool: torch.Tensor,
    block_tables: torch.Tensor,
    seq_of_token: torch.Tensor,
    positions: torch.Tensor,
    num_heads: int,
    scale: float,
    window: int | None = None,
    sink: float | torch.Tensor | None = None,
) -> None:
    """Causal attention of every token over its sequence's pages, on CUDA cores.  ``sink``: see ``_sink``.

    out [n, nh * d]; queries are the first nh * d columns of qkv; pools [pages, nkv, page_size, d];
    block_tables [seqs, max_blocks]; a token at position p reads keys max(0, p - window + 1) .. p.
    """
    _need(out, "out"), _need(qkv, "qkv", out.dtype), _need(k_pool, "k_pool", out.dtype), _need(v_pool, "v_pool", out.dtype)
    _need(block_tables, "block_tables", torch.int32), _need(seq_of_token, "seq_of_token", torch.int32)
    _need(positions, "positions", torch.int32)
    n = out.shape[0]
    _, nkv, page_size, d = k_pool.shape
    if out.dtype not in DT_CODE or out.shape[1] != num_heads * d or qkv.shape[0] != n or qkv.shape[1] < num_heads * d:
        raise KernelError("paged_attention_simt: shapes or dtype do not agree")
    if d > SIMT_MAX_HEAD_DIM or num_heads % nkv:
        raise KernelError(f"paged_attention_simt: head_dim {d} (<= {SIMT_MAX_HEAD_DIM}) / heads {num_heads} per kv head {nkv} not supported")
    f = _fn(
        "attention_simt.cu", "dli_paged_attention_simt",
        [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 6 + [c_float, c_float, c_void_p, c_int, c_void_p],
    )
    _check(
        f(_ptr(out), _ptr(qkv), qkv.shape[1], _ptr(k_pool), _ptr(v_pool), _ptr(block_tables), block_tables.shape[1],
          _ptr(seq_of_token), _ptr(positions), n, num_heads, nkv, d, page_size, int(window or 0), scale, _sink(sink), _sink_heads(sink, num_heads), DT_CODE[out.dtype], _stream()),
        "paged_attention_simt",
    )


def prefill_tc_supported(head_dim: int, page_size: int) -> bool:
    return head_dim in (64, 128) and page_size in (8, 16, 32, 64, 128)


def paged_prefill_tc(
    out: torch.Tensor,
    qkv: torch.Tensor,
    k_pool: torch.Tensor,
    v_pool: torch.Tensor,
    block_tables: torch.Tensor,
    q_start: torch.Tensor,
    kv_len: torch.Tensor,
    seq0: int,
    num_seqs: int,
    max_q_len: int,
    num_heads: int,
    scale: float,
    window: int | None = None,
    query_tiles: int = 0,
    sink: float | torch.Tensor | None = None,
) -> None:
    """bfloat16 attention for prompt portions on tcgen05 tensor cores with TMA-fed pages
    (head size 64 or 128; page sizes 8, 16, 32, 64, 128).  Arguments as paged_attention_mma.
    ``query_tiles`` (head size 64): 1 or 2 tiles of 128 (token, head) rows per CTA; 0 lets the launcher choose (two
    when a sequence brings more tokens than one tile holds)."""
    for t, name in ((out, "out"), (qkv, "qkv"), (k_pool, "k_pool"), (v_pool, "v_pool")):
        _need(t, name, torch.bfloat16)
    _need(block_tables, "block_tables", torch.int32), _need(q_start, "q_start", torch.int32), _need(kv_len, "kv_len", torch.int32)
    pages, nkv, page_size, d = k_pool.shape
    if not prefill_tc_supported(d, page_size):
        raise KernelError(f"paged_prefill_tc: head_dim {d} (64 or 128) or page size {page_size} (8..128, dividing 128) not supported")
    if out.shape[1] != num_heads * d or qkv.shape[0] != out.shape[0] or qkv.shape[1] < num_heads * d or num_heads % nkv or k_pool.shape != v_pool.shape:
        raise KernelError("paged_prefill_tc: shapes do not agree")
    if seq0 + num_seqs > kv_len.numel() or q_start.numel() != kv_len.numel() + 1:
        raise KernelError("paged_prefill_tc: sequence range outside the batch")
    f = _fn(
        "attention_tc.cu", "dli_paged_prefill_tc",
        [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 8 + [c_float, c_float, c_void_p, c_int, c_void_p],
    )
    if query_tiles not in (0, 1, 2):
        raise KernelError("paged_prefill_tc: query_tiles is 0 (choose), 1 or 2")
    _check(
        f(_ptr(out), _ptr(qkv), qkv.shape[1], _ptr(k_pool), _ptr(v_pool), pages, _ptr(block_tables), block_tables.shape[1],
          _ptr(q_start), _ptr(kv_len), seq0, num_seqs, max_q_len, num_heads, nkv, d, page_size, int(window or 0), scale, _sink(sink), _sink_heads(sink, num_heads), query_tiles, _stream()),
        "paged_prefill_tc",
    )


def decode_tma_supported(head_dim: int, page_size: int) -> bool:
    return head_dim in (64, 128) and page_size % 8 == 0 and (page_size == 8 or page_size % 16 == 0) and page_size <= 256


def paged_decode_tma(
    out: torch.Tensor,
    qkv: torch.Tensor,
    k_pool: torch.Tensor,
    v_pool: torch.Tensor,
    block_tables: torch.Tensor,
    q_start: torch.Tensor,
    kv_len: torch.Tensor,
    seq0: int,
    num_seqs: int,
    first_row: int,
    num_heads: int,
    scale: float,
    window: int | None = None,
    splits: int = 1,
    scratch: tuple[torch.Tensor, torch.Tensor] | None = None,
    max_kv_len: int = 0,
    sink: float | torch.Tensor | None = None,
) -> None:
    """bfloat16 attention of single-token sequences whose keys and values arrive by TMA (head size
    64 or 128; page sizes 8, 16, 32, ...).  Arguments as paged_attention_mma with max_q_len = 1.
    ``max_kv_len``: the longest sequence, if the host knows it (a hint: with few CTAs and long runs of keys
    the launcher gives a CTA eight warps instead of four); 0 if not."""
    for t, name in ((out, "out"), (qkv, "qkv"), (k_pool, "k_pool"), (v_pool, "v_pool")):
        _need(t, name, torch.bfloat16)
    _need(block_tables, "block_tables", torch.int32), _need(q_start, "q_start", torch.int32), _need(kv_len, "kv_len", torch.int32)
    pages, nkv, page_size, d = k_pool.shape
    if not decode_tma_supported(d, page_size):
        raise KernelError(f"paged_decode_tma: head_dim {d} (64 or 128) or page size {page_size} not supported")
    if out.shape[1] != num_heads * d or qkv.shape[0] != out.shape[0] or qkv.shape[1] < num_heads * d or num_heads % nkv or k_pool.shape != v_pool.shape:
        raise KernelError("paged_decode_tma: shapes do not agree")
    if seq0 + num_seqs > kv_len.numel() or q_start.numel() != kv_len.numel() + 1:
        raise KernelError("paged_decode_tma: sequence range outside the batch")
    acc = ml = None
    if splits > 1:
        if scratch is None:
            raise KernelError("paged_decode_tma: split keys need scratch")
        acc, ml = scratch
        _need(acc, "scratch[0]", torch.float32), _need(ml, "scratch[1]", torch.float32)
        rows = (first_row + num_seqs) * num_heads
        if acc.numel() < rows * splits * d or ml.numel() < rows * splits * 2:
            raise KernelError("paged_decode_tma: scratch too small")
    f = _fn(
        "attention_tc.cu", "dli_paged_decode_tma",
        [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 8
        + [c_float, c_float, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p],
    )
    _check(
        f(_ptr(out), _ptr(qkv), qkv.shape[1], _ptr(k_pool), _ptr(v_pool), pages, _ptr(block_tables), block_tables.shape[1],
          _ptr(q_start), _ptr(kv_len), seq0, num_seqs, first_row, num_heads, nkv, d, page_size, int(window or 0), scale, _sink(sink), _sink_heads(sink, num_heads),
          splits, _ptr(acc), _ptr(ml), int(max_kv_len), _stream()),
        "paged_decode_tma",
    )
    global launch_count
    if splits > 1 and not _fn("attention_tc.cu", "dli_decode_tma_merges_in_cluster", [c_int, c_int, c_int])(num_heads, nkv, splits):
        launch_count += 1  # the merge kernel; otherwise the splits merge inside the kernel, as one cluster


def paged_prefill_tc_error() -> int:
    """0, or which bounded wait of the tcgen05 / TMA attention kernels ran out since the library was loaded
    (or since the code was last cleared)."""
    return _fn("attention_tc.cu", "dli_paged_prefill_tc_error", [])()


def _library_in_use(source: str) -> bool:
    return any(key.startswith(source + ":") for key in _fns)


def device_wait_errors(clear: bool = True) -> dict[str, int]:
    """Bounded device waits that ran out: {library: code} for the libraries this process has used
    (a library nobody called has recorded nothing and is not built for the question).  The flags live
    in mapped host memory, so reading them costs no copy; read them once the step's results have
    reached the host.  With ``clear`` a code that was read is forgotten."""
    found = {}
    for source, read, forget in (("skinny_gemm.cu", "dli_skinny_gemm_error", "dli_skinny_gemm_clear_error"),
                                 ("dense_gemm.cu", "dli_dense_gemm_error", "dli_dense_gemm_clear_error"),
                                 ("attention_tc.cu", "dli_paged_prefill_tc_error", "dli_paged_prefill_tc_clear_error")):
        if not _library_in_use(source):
            continue
        code = _fn(source, read, [])()
        if code:
            found[source] = int(code)
            if clear:
                _fn(source, forget, [])()
    return found


# ------------------------------------------------------------------ sampling


# A stochastic row's logits are kept in the shared memory of a cluster of 8 CTAs, 47 K floats each
SAMPLE_MAX_VOCAB_STOCHASTIC = 8 * 47 * 1024


def sample(
    out: torch.Tensor,
    logits: torch.Tensor,
    temperature: torch.Tensor | None = None,
    top_k: torch.Tensor | None = None,
    top_p: torch.Tensor | None = None,
    seed: torch.Tensor | None = None,
    draw: torch.Tensor | None = None,
    slots: torch.Tensor | None = None,
) -> None:
    """out[r] = token of row r of float32 logits [rows, V]; all-greedy when temperature is None.
    seed and draw are int64 tensors read as unsigned 64-bit.  With ``slots`` (int32, one per row) the five
    parameter tensors are tables indexed by slots[r] instead of r (the requests' state slots), and the draw
    count of every stochastic row's slot is advanced by one on the device."""
    _need(out, "out", torch.int32), _need(logits, "logits", torch.float32)
    rows, V = logits.shape
    if out.numel() != rows:
        raise KernelError("sample: one output per row")
    if temperature is not None:
        if top_k is None or top_p is None or seed is None or draw is None:
            raise KernelError("sample: stochastic rows need top_k, top_p, seed and draw")
        if V > SAMPLE_MAX_VOCAB_STOCHASTIC:
            raise KernelError(f"sample: temperature sampling takes vocabularies of up to {SAMPLE_MAX_VOCAB_STOCHASTIC} tokens, not {V} "
                              "(greedy rows alone, passed without parameters, take any)")
        _need(temperature, "temperature", torch.float32), _need(top_k, "top_k", torch.int32), _need(top_p, "top_p", torch.float32)
        _need(seed, "seed", torch.int64), _need(draw, "draw", torch.int64)
        entries = rows if slots is None else temperature.numel()
        if not (temperature.numel() == top_k.numel() == top_p.numel() == seed.numel() == draw.numel() == entries):
            raise KernelError("sample: one parameter per row (or, with slots, tables of one length)")
    if slots is not None:
        _need(slots, "slots", torch.int32)
        if temperature is None or slots.numel() != rows:
            raise KernelError("sample: slots go with parameter tables and name one slot per row")
    f = _fn(
        "sampling.cu", "dli_sample",
        [c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    )
    _check(
        f(_ptr(out), _ptr(logits), logits.stride(0), rows, V, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(seed), _ptr(draw), _ptr(slots),
          _stream()),
        "sample",
    )


def mma_head_dim_supported(head_dim: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= 256


def paged_attention_mma(
    out: torch.Tensor,
    qkv: torch.Tensor,
    k_pool: torch.Tensor,
    v_pool: torch.Tensor,
    block_tables: torch.Tensor,
    q_start: torch.Tensor,
    kv_len: torch.Tensor,
    seq0: int,
    num_seqs: int,
    max_q_len: int,
    first_row: int,
    num_heads: int,
    scale: float,
    window: int | None = None,
    splits: int = 1,
    scratch: tuple[torch.Tensor, torch.Tensor] | None = None,
    sink: float | torch.Tensor | None = None,
) -> None:
    """bfloat16 tensor-core attention for the sequences [seq0, seq0 + num_seqs) of a batch.

    Queries are the first nh * d columns of qkv; a sequence's tokens sit in rows
    q_start[s] .. q_start[s + 1] at positions kv_len[s] - q_len .. kv_len[s] - 1.  With
    ``splits`` > 1 (single-token sequences only) the keys are cut into that many runs;
    ``scratch`` = (float32 [rows * splits * d], float32 [rows * splits * 2]) with
    rows = (first_row + num_seqs) * nh holds the partial results.
    """
    for t, name in ((out, "out"), (qkv, "qkv"), (k_pool, "k_pool"), (v_pool, "v_pool")):
        _need(t, name, torch.bfloat16)
    _need(block_tables, "block_tables", torch.int32), _need(q_start, "q_start", torch.int32), _need(kv_len, "kv_len", torch.int32)
    _, nkv, page_size, d = k_pool.shape
    if not mma_head_dim_supported(d):
        raise KernelError(f"paged_attention_mma: head_dim {d} is not a multiple of 16 in [16, 256]")
    if out.shape[1] != num_heads * d or qkv.shape[0] != out.shape[0] or qkv.shape[1] < num_heads * d or num_heads % nkv:
        raise KernelError("paged_attention_mma: shapes do not agree")
    if seq0 + num_seqs > kv_len.numel() or q_start.numel() != kv_len.numel() + 1:
        raise KernelError("paged_attention_mma: sequence range outside the batch")
    acc = ml = None
    if splits > 1:
        if max_q_len != 1 or scratch is None:
            raise KernelError("paged_attention_mma: split keys need single-token sequences and scratch")
        acc, ml = scratch
        _need(acc, "scratch[0]", torch.float32), _need(ml, "scratch[1]", torch.float32)
        rows = (first_row + num_seqs) * num_heads
        if acc.numel() < rows * splits * d or ml.numel() < rows * splits * 2:
            raise KernelError("paged_attention_mma: scratch too small")
    f = _fn(
        "attention_mma.cu", "dli_paged_attention_mma",
        [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]
        + [c_int] * 8 + [c_float, c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p],
        {"HEAD_DIM": d},
    )
    _check(
        f(_ptr(out), _ptr(qkv), qkv.shape[1], _ptr(k_pool), _ptr(v_pool), _ptr(block_tables), block_tables.shape[1],
          _ptr(q_start), _ptr(kv_len), seq0, num_seqs, max_q_len, first_row, num_heads, nkv, page_size, int(window or 0),
          scale, _sink(sink), _sink_heads(sink, num_heads), splits, _ptr(acc), _ptr(ml), _stream()),
        "paged_attention_mma",
    )
    global launch_count
    if splits > 1:
        launch_count += 1  # the merge kernel


# ------------------------------------------------------------------ decode matrix product


def skinny_gemm_supported(tokens: int, in_features: int) -> bool:
    return 1 <= tokens <= 256 and in_features >= 8 and in_features % 8 == 0


class ScaledRows:
    """Activations whose rows still lack a factor: ``x`` [n, size] holds bfloat16(h * gain) of a
    residual stream h, ``ssq`` [n, tiles] float32 the sums of h^2 over tiles of 128 features, and
    the finished RMS norm is x[t] * rsqrt(sum(ssq[t]) / size + eps).  A factor per row commutes
    with a matrix product, so the decode products take this as their input and apply the factor
    to their float32 sums (``skinny_gemm*``); ``skinny_gemm_residual`` makes it."""

    __slots__ = ("x", "ssq", "eps")

    def __init__(self, x: torch.Tensor, ssq: torch.Tensor, eps: float) -> None:
        self.x, self.ssq, self.eps = x, ssq, float(eps)

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype

    @property
    def device(self):
        return self.x.device


def _row_scale(x, name: str):
    """(activations, the four row-scaling arguments of the kernel) for a tensor or ScaledRows."""
    if not isinstance(x, ScaledRows):
        return x, (None, 0, 0.0, 0)
    _need(x.ssq, name + ".ssq", torch.float32)
    n, size = x.x.shape
    if x.ssq.dim() != 2 or x.ssq.shape[0] != n or n > 64:
        raise KernelError(f"{name}: row sums of squares must be [tokens <= 64, tiles]")
    return x.x, (_ptr(x.ssq), x.ssq.shape[1], x.eps, size)


_ROW_SCALE_ARGS = [c_void_p, c_int, c_float, c_int]
_slices_cache: dict[tuple[int, int, int], int] = {}


def skinny_gemm_slices(tokens: int, features: int, in_features: int) -> int:
    """K slices the kernel's launcher recommends for these sizes."""
    key = (tokens, features, in_features)
    n = _slices_cache.get(key)
    if n is None:
        n = _slices_cache[key] = _fn("skinny_gemm.cu", "dli_skinny_gemm_slices", [c_int, c_int, c_int])(*key)
    return n


def skinny_gemm(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, slices: int | None = None,
                out: torch.Tensor | None = None, max_stages: int = 0) -> torch.Tensor:
    """x [tokens <= 256, K] times weight [features, K] transposed, bfloat16 in, on tcgen05 tensor
    cores fed by TMA; returns [tokens, features] in bfloat16 or float32.  ``slices`` (1..16) cuts K
    across the CTAs of a cluster, which add their partial sums through distributed shared memory."""
    x, scale = _row_scale(x, "skinny_gemm")
    _need(x, "x", torch.bfloat16), _need(weight, "weight", torch.bfloat16)
    tokens, K = x.shape
    features = weight.shape[0]
    if weight.shape[1] != K or not skinny_gemm_supported(tokens, K) or out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"skinny_gemm: tokens {tokens} (1..256), K {K} (a multiple of 8) or output {out_dtype} not supported")
    if slices is not None and not 1 <= slices <= 16:
        raise KernelError("skinny_gemm: 1 to 16 K slices")
    if slices is None:
        slices = skinny_gemm_slices(tokens, features, K)
    if out is None:
        out = torch.empty((tokens, features), dtype=out_dtype, device=x.device)
    else:
        _need(out, "out", out_dtype)
        if tuple(out.shape) != (tokens, features):
            raise KernelError("skinny_gemm: out has the wrong shape")
    f = _fn("skinny_gemm.cu", "dli_skinny_gemm", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int] + _ROW_SCALE_ARGS + [c_void_p])
    _check(f(_ptr(out), int(out_dtype == torch.float32), _ptr(x), _ptr(weight), tokens, features, K, slices, max_stages, *scale, _stream()), "skinny_gemm")
    return out


def skinny_gemm_wait_test(x: torch.Tensor, weight: torch.Tensor, slices: int, wait_limit: int, skip_tile: int) -> torch.Tensor:
    """For the test of the kernel's bounded waits: the plain product in float32, except that the copies of k tile
    ``skip_tile`` (64 columns of K each) are left out and every wait gives up after ``wait_limit`` polls.  The
    kernel then records code 2 (``skinny_gemm_error``), stores what it has and returns; nothing hangs or
    faults.  ``skip_tile`` must be the last tile of its slice and K / 64 / slices at most 8.  Not used by the engine."""
    _need(x, "x", torch.bfloat16), _need(weight, "weight", torch.bfloat16)
    tokens, K = x.shape
    features = weight.shape[0]
    per = -(-(-(-K // 64)) // slices)
    if weight.shape[1] != K or not 1 <= slices <= 16 or per > 8 or skip_tile < 0 or (skip_tile + 1) % per:
        raise KernelError("skinny_gemm_wait_test: the tile left out must be the last one of a slice of at most 8 tiles")
    out = torch.zeros((tokens, features), dtype=torch.float32, device=x.device)
    f = _fn("skinny_gemm.cu", "dli_skinny_gemm_wait_test", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, ctypes.c_uint, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(x), _ptr(weight), tokens, features, K, slices, wait_limit, skip_tile, _stream()), "skinny_gemm_wait_test")
    return out


def skinny_gemm_residual(x, weight: torch.Tensor, h: torch.Tensor, gain: torch.Tensor, eps: float, slices: int | None = None) -> ScaledRows:
    """h += x W^T (float32, in place) and the first half of the RMS norm that follows, in the
    product's epilogue: returns ScaledRows(bfloat16(h * gain), sums of h^2 per 128 features, eps).
    x [tokens <= 64, K] may itself be ScaledRows."""
    x, scale = _row_scale(x, "skinny_gemm_residual")
    _need(x, "x", torch.bfloat16), _need(weight, "weight", torch.bfloat16), _need(h, "h", torch.float32), _need(gain, "gain", torch.float32)
    tokens, K = x.shape
    features = weight.shape[0]
    if weight.shape[1] != K or not skinny_gemm_supported(tokens, K) or tokens > 64:
        raise KernelError(f"skinny_gemm_residual: tokens {tokens} (1..64) or K {K} (a multiple of 8) not supported")
    if tuple(h.shape) != (tokens, features) or gain.numel() != features:
        raise KernelError("skinny_gemm_residual: h must be [tokens, features] and gain [features]")
    if slices is None:
        slices = skinny_gemm_slices(tokens, features, K)
    out = torch.empty((tokens, features), dtype=torch.bfloat16, device=x.device)
    ssq = torch.empty((tokens, (features + 127) // 128), dtype=torch.float32, device=x.device)
    f = _fn("skinny_gemm.cu", "dli_skinny_gemm_residual",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int] + _ROW_SCALE_ARGS + [c_void_p])
    _check(f(_ptr(out), _ptr(h), _ptr(gain), _ptr(ssq), _ptr(x), _ptr(weight), tokens, features, K, slices, *scale, _stream()), "skinny_gemm_residual")
    return ScaledRows(out, ssq, eps)


def skinny_gemm_swiglu(x: torch.Tensor, weight_tiled: torch.Tensor, activation: str = "silu", limit: float = 0.0, up_shift: float = 0.0) -> torch.Tensor:
    """act(x Wg^T) * (x Wu^T) (act: silu or another of GLU_ACTIVATIONS; bounds and shift as in ``silu_mul``) in one kernel: the decode matrix
    product with the activation in its epilogue.  weight_tiled [2 I, K]: rows in blocks of 128 — 64 gate rows, then the 64 up rows of
    the same features.  Returns bfloat16 [tokens, I]."""
    x, scale = _row_scale(x, "skinny_gemm_swiglu")
    _need(x, "x", torch.bfloat16), _need(weight_tiled, "weight", torch.bfloat16)
    tokens, K = x.shape
    features = weight_tiled.shape[0]
    if weight_tiled.shape[1] != K or features % 128 or not skinny_gemm_supported(tokens, K) or activation not in GLU_ACTIVATIONS:
        raise KernelError("skinny_gemm_swiglu: sizes or activation not supported")
    out = torch.empty((tokens, features // 2), dtype=torch.bfloat16, device=x.device)
    f = _fn("skinny_gemm.cu", "dli_skinny_gemm_swiglu", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float] + _ROW_SCALE_ARGS + [c_void_p])
    _check(f(_ptr(out), _ptr(x), _ptr(weight_tiled), tokens, features, K, skinny_gemm_slices(tokens, features, K), GLU_ACTIVATIONS[activation],
             float(limit), float(up_shift), *scale, _stream()), "skinny_gemm_swiglu")
    return out


def skinny_gemm_act(x, weight: torch.Tensor, kind: str) -> torch.Tensor:
    """act(x W^T) in one kernel: the decode matrix product with the activation of a plain feed-forward (``relu2``,
    ``gelu_tanh``, ``silu``) in its epilogue, applied to the sums rounded to bfloat16 (what the product alone would have
    stored).  Returns bfloat16 [tokens, features]."""
    x, scale = _row_scale(x, "skinny_gemm_act")
    _need(x, "x", torch.bfloat16), _need(weight, "weight", torch.bfloat16)
    tokens, K = x.shape
    features = weight.shape[0]
    if weight.shape[1] != K or not skinny_gemm_supported(tokens, K) or kind not in ACTIVATIONS:
        raise KernelError("skinny_gemm_act: sizes or activation not supported")
    out = torch.empty((tokens, features), dtype=torch.bfloat16, device=x.device)
    f = _fn("skinny_gemm.cu", "dli_skinny_gemm_act", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int] + _ROW_SCALE_ARGS + [c_void_p])
    _check(f(_ptr(out), _ptr(x), _ptr(weight), tokens, features, K, skinny_gemm_slices(tokens, features, K), ACTIVATIONS[kind] + 1, *scale, _stream()),
           "skinny_gemm_act")
    return out


def skinny_rotary_supported(head_dim: int) -> bool:
    return head_dim >= 2 and 128 % head_dim == 0


def skinny_gemm_rotary(x, wqkv, positions, inv_freq, slots, k_pool, v_pool, num_heads: int, num_kv_heads: int, head_dim: int,
                       rotary_dim: int, page_size: int, write_kv: bool) -> torch.Tensor:
    """q | k | v = x Wqkv^T with the rotary embedding and the write of keys and values into the
    cache pages done in the product's epilogue; returns the rotated queries [tokens, nh * d]."""
    x, scale = _row_scale(x, "skinny_gemm_rotary")
    _need(x, "x", torch.bfloat16), _need(wqkv, "wqkv", torch.bfloat16), _need(positions, "positions", torch.int32)
    tokens, K = x.shape
    features = (num_heads + 2 * num_kv_heads) * head_dim
    if tuple(wqkv.shape) != (features, K) or not skinny_gemm_supported(tokens, K) or not skinny_rotary_supported(head_dim):
        raise KernelError("skinny_gemm_rotary: sizes not supported")
    if rotary_dim:
        _need(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("skinny_gemm_rotary: inv_freq must have rotary_dim / 2 entries")
    if write_kv:
        _need(slots, "slots", torch.int32), _need(k_pool, "k_pool", torch.bfloat16), _need(v_pool, "v_pool", torch.bfloat16)
        if tuple(k_pool.shape[1:]) != (num_kv_heads, page_size, head_dim) or k_pool.shape != v_pool.shape or slots.numel() != tokens:
            raise KernelError("skinny_gemm_rotary: pool layout must be [pages, kv_heads, page_size, head_dim]")
    q = torch.empty((tokens, num_heads * head_dim), dtype=torch.bfloat16, device=x.device)
    f = _fn("skinny_gemm.cu", "dli_skinny_gemm_rotary",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 6
            + _ROW_SCALE_ARGS + [c_void_p])
    _check(f(_ptr(q), _ptr(x), _ptr(wqkv), tokens, K, skinny_gemm_slices(tokens, features, K), _ptr(positions),
             _ptr(inv_freq if rotary_dim else None), _ptr(slots if write_kv else None), _ptr(k_pool if write_kv else None),
             _ptr(v_pool if write_kv else None), num_heads, num_kv_heads, head_dim, rotary_dim, page_size, int(write_kv), *scale, _stream()),
           "skinny_gemm_rotary")
    return q


# ------------------------------------------------------------------ matrix product of many tokens
# A portion of a prompt: tokens are the 128-row side of the tensor-core instruction, a thread of the epilogue holds
# one token's row of a tile, and the elementwise step behind the product is done on the sums before they are stored.


def dense_gemm_supported(in_features: int, features: int) -> bool:
    return in_features >= 8 and in_features % 8 == 0 and features >= 8 and features % 8 == 0


def dense_rotary_supported(head_dim: int, rotary_dim: int) -> bool:
    return head_dim in (64, 128) and rotary_dim in (0, 64, 128) and rotary_dim <= head_dim


def _dense_sizes(x: torch.Tensor, weight: torch.Tensor, name: str):
    _need(x, "x", torch.bfloat16), _need(weight, "weight", torch.bfloat16)
    tokens, K = x.shape
    features = weight.shape[0]
    if weight.shape[1] != K or tokens < 1 or not dense_gemm_supported(K, features):
        raise KernelError(f"{name}: K {K} and features {features} must be multiples of 8 and the shapes agree")
    return tokens, features, K


def dense_gemm(x, weight: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """x [tokens, K] times weight [features, K] transposed, bfloat16 in and out, float32 sums, on tcgen05 tensor
    cores fed by TMA: persistent pairs of CTAs (cta_group::2) over tiles of 256 tokens x 256 features, two
    accumulators in each CTA's tensor memory."""
    tokens, features, K = _dense_sizes(x, weight, "dense_gemm")
    if out is None:
        out = torch.empty((tokens, features), dtype=torch.bfloat16, device=x.device)
    else:
        _need(out, "out", torch.bfloat16)
        if tuple(out.shape) != (tokens, features):
            raise KernelError("dense_gemm: out has the wrong shape")
    f = _fn("dense_gemm.cu", "dli_dense_gemm", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(x), _ptr(weight), tokens, features, K, _stream()), "dense_gemm")
    return out


def dense_gemm_act(x, weight: torch.Tensor, kind: str) -> torch.Tensor:
    """act(x W^T) in the product's epilogue (``relu2``, ``gelu_tanh``, ``silu``), applied to the sums rounded to bfloat16.
    Returns bfloat16 [tokens, features]."""
    tokens, features, K = _dense_sizes(x, weight, "dense_gemm_act")
    if kind not in ACTIVATIONS:
        raise KernelError(f"dense_gemm_act: activation {kind!r} not supported")
    out = torch.empty((tokens, features), dtype=torch.bfloat16, device=x.device)
    f = _fn("dense_gemm.cu", "dli_dense_gemm_act", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(x), _ptr(weight), tokens, features, K, ACTIVATIONS[kind] + 1, _stream()), "dense_gemm_act")
    return out


def dense_gemm_swiglu(x, weight_tiled: torch.Tensor, activation: str = "silu", limit: float = 0.0, up_shift: float = 0.0) -> torch.Tensor:
    """act(x Wg^T) * (x Wu^T) (act: silu or another of GLU_ACTIVATIONS; bounds and shift as in ``silu_mul``) in the product's epilogue.  weight_tiled [2 I, K]: rows in blocks of 128 — 64 gate
    rows, then the 64 up rows of the same features.  Returns bfloat16 [tokens, I]."""
    tokens, features, K = _dense_sizes(x, weight_tiled, "dense_gemm_swiglu")
    if features % 128 or activation not in GLU_ACTIVATIONS:
        raise KernelError("dense_gemm_swiglu: the interleaved layout needs an intermediate size that is a multiple of 64, and a known activation")
    act = torch.empty((tokens, features // 2), dtype=torch.bfloat16, device=x.device)
    f = _fn("dense_gemm.cu", "dli_dense_gemm_swiglu", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p])
    _check(f(_ptr(act), _ptr(x), _ptr(weight_tiled), tokens, features, K, GLU_ACTIVATIONS[activation], float(limit), float(up_shift), _stream()),
           "dense_gemm_swiglu")
    return act


def dense_gemm_rotary(x, wqkv, table, slots, k_pool, v_pool, num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int,
                      page_size: int, write_kv: bool) -> torch.Tensor:
    """q | k | v = x Wqkv^T with the rotary embedding (``table`` [tokens, rotary_dim]: cos | sin of every token's
    angles, as ``rotary_table`` makes it) and the write of keys and values into the cache pages done in the
    product's epilogue; returns the rotated queries [tokens, nh * d]."""
    features = (num_heads + 2 * num_kv_heads) * head_dim
    tokens, _, K = _dense_sizes(x, wqkv, "dense_gemm_rotary")
    if wqkv.shape[0] != features or not dense_rotary_supported(head_dim, rotary_dim):
        raise KernelError("dense_gemm_rotary: sizes not supported")
    if rotary_dim:
        _need(table, "table", torch.float32)
        if tuple(table.shape) != (tokens, rotary_dim):
            raise KernelError("dense_gemm_rotary: table must be [tokens, rotary_dim]")
    if write_kv:
        _need(slots, "slots", torch.int32), _need(k_pool, "k_pool", torch.bfloat16), _need(v_pool, "v_pool", torch.bfloat16)
        if tuple(k_pool.shape[1:]) != (num_kv_heads, page_size, head_dim) or k_pool.shape != v_pool.shape or slots.numel() != tokens:
            raise KernelError("dense_gemm_rotary: pool layout must be [pages, kv_heads, page_size, head_dim]")
    q = torch.empty((tokens, num_heads * head_dim), dtype=torch.bfloat16, device=x.device)
    f = _fn("dense_gemm.cu", "dli_dense_gemm_rotary",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 6 + [c_void_p])
    _check(f(_ptr(q), _ptr(x), _ptr(wqkv), tokens, K, _ptr(table if rotary_dim else None), _ptr(slots if write_kv else None),
             _ptr(k_pool if write_kv else None), _ptr(v_pool if write_kv else None), num_heads, num_kv_heads, head_dim, rotary_dim,
             page_size, int(write_kv), _stream()), "dense_gemm_rotary")
    return q


def dense_gemm_wait_test(x: torch.Tensor, weight: torch.Tensor, wait_limit: int) -> torch.Tensor:
    """For the test of the kernel's bounded waits: the product of one tile (tokens <= 256, features <= 256, K <= 384)
    in which neither CTA of the pair issues the copies of the last k step and every wait gives up after
    ``wait_limit`` polls.  The kernel records a code (``dense_gemm_error``: 3, the wait for operands, or 4, the wait
    for the accumulator that depends on them), both CTAs end together and free their tensor memory; nothing hangs or
    faults.  Not used by the engine."""
    tokens, features, K = _dense_sizes(x, weight, "dense_gemm_wait_test")
    out = torch.zeros((tokens, features), dtype=torch.bfloat16, device=x.device)
    f = _fn("dense_gemm.cu", "dli_dense_gemm_wait_test", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, ctypes.c_uint, c_void_p])
    _check(f(_ptr(out), _ptr(x), _ptr(weight), tokens, features, K, int(wait_limit), _stream()), "dense_gemm_wait_test")
    return out


def dense_gemm_error() -> int:
    """0, or which bounded wait of the many-token product ran out (1 copies, 2 and 3 products, 4 epilogue)."""
    return _fn("dense_gemm.cu", "dli_dense_gemm_error", [])()


def skinny_gemm_error() -> int:
    """0, or which bounded wait of the decode matrix product ran out since the library was loaded."""
    return _fn("skinny_gemm.cu", "dli_skinny_gemm_error", [])()


# ------------------------------------------------------------------ layer norm around the residual stream


def post_add_layernorm(y: torch.Tensor | None, h: torch.Tensor, a: torch.Tensor | None, w_post: torch.Tensor | None,
                       w_pre: torch.Tensor | None, eps_post: float, eps_pre: float, rows: torch.Tensor | None = None) -> None:
    """Layer norm (weight, no bias) on both sides of the residual addition, in one kernel:

        v = h[s] + LN(a[s]) * w_post     (the addition is skipped when ``a`` is None)
        y[r] = LN(v) * w_pre             (skipped when ``y`` is None)

    with s = rows[r] (or r).  Without ``rows`` v is written back to ``h``.  LN(x) = (x - mean) / sqrt(var + eps),
    var the mean of the squared deviations; all in float32."""
    _need(h, "h", torch.float32)
    n, H = h.shape
    dtype = y.dtype if y is not None else (a.dtype if a is not None else None)
    if dtype not in DT_CODE:
        raise KernelError("post_add_layernorm: nothing to do, or a dtype that is not supported")
    if a is not None:
        _need(a, "a", dtype), _need(w_post, "w_post", torch.float32)
        if a.shape != h.shape or w_post.numel() != H:
            raise KernelError("post_add_layernorm: a and h differ in shape, or w_post is not [H]")
    n_rows = n
    if rows is not None:
        _need(rows, "rows", torch.int32)
        n_rows = rows.numel()
    if y is not None:
        _need(y, "y"), _need(w_pre, "w_pre", torch.float32)
        if tuple(y.shape) != (n_rows, H) or w_pre.numel() != H:
            raise KernelError("post_add_layernorm: y must be [rows, H] and w_pre [H]")
    f = _fn("layernorm.cu", "dli_post_add_layernorm",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_int, c_void_p])
    _check(f(_ptr(y), _ptr(h), _ptr(a), _ptr(w_post), _ptr(w_pre), _ptr(rows), n_rows, H, eps_post, eps_pre, DT_CODE[dtype], _stream()),
           "post_add_layernorm")


def stream_reinject(h: torch.Tensor, table: torch.Tensor | None, ids: torch.Tensor | None, vec: torch.Tensor | None) -> None:
    """h[t] += table[ids[t]] + vec: the embedding of the step's tokens (if ``table``) and one vector (if ``vec``) are
    added to the float32 residual stream."""
    _need(h, "h", torch.float32)
    n, H = h.shape
    code = DT_CODE[torch.float32]
    if table is not None:
        _need(table, "table"), _need(ids, "ids", torch.int32)
        if table.dtype not in DT_CODE or table.shape[1] != H or ids.numel() != n:
            raise KernelError("stream_reinject: shapes or dtype do not agree")
        code = DT_CODE[table.dtype]
    if vec is not None:
        _need(vec, "vec", torch.float32)
        if vec.numel() != H:
            raise KernelError("stream_reinject: vec must be [H]")
    f = _fn("layernorm.cu", "dli_stream_reinject", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(h), _ptr(table), _ptr(ids), _ptr(vec), n, H, code, _stream()), "stream_reinject")


def activation(x: torch.Tensor, kind: str) -> torch.Tensor:
    """x <- act(x) in place and returned: ``relu2`` (the square of relu), ``gelu_tanh``, ``silu``, ``tanh``."""
    _need(x, "x")
    if x.dtype not in DT_CODE or kind not in ELEMENTWISE_ACTIVATIONS:
        raise KernelError(f"activation: dtype {x.dtype} or kind {kind!r} (known: {sorted(ELEMENTWISE_ACTIVATIONS)}) not supported")
    f = _fn("elementwise.cu", "dli_activation", [c_void_p, c_longlong, c_int, c_int, c_void_p])
    _check(f(_ptr(x), x.numel(), ELEMENTWISE_ACTIVATIONS[kind], DT_CODE[x.dtype], _stream()), "activation")
    return x


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2}  # what a plain feed-forward may use (also in the products' epilogues)
ELEMENTWISE_ACTIVATIONS = {**ACTIVATIONS, "tanh": 3}  # what the kernel of its own takes


# ------------------------------------------------------------------ between an attention mixer's projections and its kernel


def qk_norm_rotary_store(proj: torch.Tensor, wq: torch.Tensor | None, wk: torch.Tensor | None, eps: float, positions: torch.Tensor,
                         inv_freq: torch.Tensor | None, slots: torch.Tensor | None, k_pool: torch.Tensor | None,
                         v_pool: torch.Tensor | None, num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int,
                         page_size: int, write_kv: bool = True, values_from_keys: bool = True) -> torch.Tensor:
    """proj [n, >= (nh + nkv) d]: q | k (| v, when the values are not the keys) as projected.  With ``wq`` and ``wk``
    q and k are each divided by the RMS of the whole projection (all heads together, ``eps`` inside the root) and
    multiplied by these weights [nh d], [nkv d]; then rotary (rotate-half pairing) on the first ``rotary_dim``
    dimensions of every head.  Returns q [n, nh d]; k goes to ``k_pool`` and the values — the keys as projected
    (``values_from_keys``) or the columns behind k — to ``v_pool`` [pages, nkv, page_size, d] at ``slots``."""
    _need(positions, "positions", torch.int32)
    if proj.dtype not in DT_CODE or proj.dim() != 2 or proj.stride(1) != 1 or not proj.is_cuda:
        raise KernelError("qk_norm_rotary_store: proj must be a CUDA matrix with unit column stride")
    n = proj.shape[0]
    need_cols = (num_heads + (1 if values_from_keys else 2) * num_kv_heads) * head_dim
    if proj.shape[1] < need_cols or positions.numel() != n:
        raise KernelError("qk_norm_rotary_store: shapes do not agree")
    normed = wq is not None
    if normed:
        _need(wq, "wq", torch.float32), _need(wk, "wk", torch.float32)
        if wq.numel() != num_heads * head_dim or wk.numel() != num_kv_heads * head_dim:
            raise KernelError("qk_norm_rotary_store: norm weights must cover the whole projections")
    if rotary_dim:
        _need(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("qk_norm_rotary_store: inv_freq must have rotary_dim / 2 entries")
    if write_kv:
        _need(slots, "slots", torch.int32), _need(k_pool, "k_pool", proj.dtype), _need(v_pool, "v_pool", proj.dtype)
        if tuple(k_pool.shape[1:]) != (num_kv_heads, page_size, head_dim) or k_pool.shape != v_pool.shape or slots.numel() != n:
            raise KernelError("qk_norm_rotary_store: pool layout must be [pages, kv_heads, page_size, head_dim]")
    q = torch.empty((n, num_heads * head_dim), dtype=proj.dtype, device=proj.device)
    f = _fn("attention_prep.cu", "dli_qk_norm_rotary_store",
            [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 10 + [c_void_p])
    _check(f(_ptr(q), _ptr(proj), proj.stride(0), _ptr(wq), _ptr(wk), eps, _ptr(positions), _ptr(inv_freq if rotary_dim else None),
             _ptr(slots if write_kv else None), _ptr(k_pool if write_kv else None), _ptr(v_pool if write_kv else None), n, num_heads,
             num_kv_heads, head_dim, rotary_dim, page_size, int(write_kv), int(normed), int(values_from_keys), DT_CODE[proj.dtype], _stream()),
           "qk_norm_rotary_store")
    return q


def sigmoid_gate(out: torch.Tensor, gate: torch.Tensor) -> None:
    """out *= sigmoid(gate), element by element; ``gate`` [n, cols] may be a column slice of a wider matrix."""
    _need(out, "out")
    n, cols = out.shape
    if out.dtype not in DT_CODE or gate.dtype != out.dtype or tuple(gate.shape) != (n, cols) or gate.stride(1) != 1 or not gate.is_cuda:
        raise KernelError("sigmoid_gate: shapes or dtype do not agree")
    f = _fn("attention_prep.cu", "dli_sigmoid_gate", [c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(out), c_void_p(gate.data_ptr()), gate.stride(0), n, cols, DT_CODE[out.dtype], _stream()), "sigmoid_gate")


def latent_prep(q_out: torch.Tensor, proj: torch.Tensor, w_norm: torch.Tensor, eps: float, positions: torch.Tensor,
                inv_freq: torch.Tensor | None, slots: torch.Tensor | None, k_pool: torch.Tensor | None, num_heads: int, head_dim: int,
                rot_dim: int, kv_rank: int, rotary_dim: int, page_size: int, amp: float = 1.0) -> None:
    """Between the projections of an attention over a cached latent and its attention kernel, one kernel a step.
    proj [n, >= nh (d + dr) + r + dr]: per head d plain and dr rotated query numbers, then the down projection: r latent
    numbers and dr of a key part that all heads share.  The latent is divided by its RMS (``eps`` inside the root) and
    multiplied by ``w_norm`` [r]; the first ``rotary_dim`` of the dr numbers of the key part and of every head's query part
    are rotated (rotate-half pairing, angle float32(position) * inv_freq[i], cosines and sines times ``amp``).  The cache row latent | key part goes to
    ``k_pool`` [pages, 1, page_size, r + dr] at ``slots`` (if given); the rotated query parts go to columns r .. r + dr of
    every head of ``q_out`` [n, nh (r + dr)], whose other columns this kernel leaves alone."""
    _need(positions, "positions", torch.int32), _need(q_out, "q_out"), _need(w_norm, "w_norm", torch.float32)
    if proj.dtype not in DT_CODE or proj.dim() != 2 or proj.stride(1) != 1 or not proj.is_cuda or q_out.dtype != proj.dtype:
        raise KernelError("latent_prep: proj must be a CUDA matrix with unit column stride, q_out of its dtype")
    n = proj.shape[0]
    row = kv_rank + rot_dim
    if (proj.shape[1] < num_heads * (head_dim + rot_dim) + row or positions.numel() != n or tuple(q_out.shape) != (n, num_heads * row)
            or w_norm.numel() != kv_rank or rotary_dim % 2 or rotary_dim > rot_dim):
        raise KernelError("latent_prep: shapes do not agree")
    if rotary_dim:
        _need(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("latent_prep: inv_freq must have rotary_dim / 2 entries")
    write = slots is not None
    if write:
        _need(slots, "slots", torch.int32), _need(k_pool, "k_pool", proj.dtype)
        if tuple(k_pool.shape[1:]) != (1, page_size, row) or slots.numel() != n:
            raise KernelError("latent_prep: pool layout must be [pages, 1, page_size, kv_rank + rot_dim]")
    f = _fn("attention_prep.cu", "dli_latent_prep",
            [c_void_p, c_void_p, c_longlong, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 7 + [c_float, c_int, c_void_p])
    _check(f(_ptr(q_out), _ptr(proj), proj.stride(0), _ptr(w_norm), eps, _ptr(positions), _ptr(inv_freq if rotary_dim else None),
             _ptr(slots if write else None), _ptr(k_pool if write else None), n, num_heads, head_dim, rot_dim, kv_rank, rotary_dim, page_size,
             float(amp), DT_CODE[proj.dtype], _stream()), "latent_prep")


def rotary_unit_store(q_out: torch.Tensor, x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor | None, slots: torch.Tensor | None,
                      k_pool: torch.Tensor | None, v_pool: torch.Tensor | None, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                      rotary_dim: int, unit_eps: float | None, page_size: int) -> None:
    """Between an attention mixer's convolutions and its attention kernel, one kernel a step.  x [n, (nh + nkv) d + nkv dv]: q | k | v.
    Every q and k head is rotated on its first ``rotary_dim`` dimensions (rotate-half pairing, angle float32(position) *
    inv_freq[i]) and then, unless ``unit_eps`` is None, divided by sqrt(mean(head^2) + unit_eps); float32 throughout, one rounding.
    Rows of D = max(d, dv) numbers leave, the shorter of keys and values padded with zeros: q to ``q_out`` [n, nh D], k and v to
    the pools [pages, nkv, page_size, D] at ``slots`` (if given)."""
    _need(positions, "positions", torch.int32), _need(q_out, "q_out"), _need(x, "x", q_out.dtype)
    n = x.shape[0]
    D = max(head_dim, value_dim)
    if (x.dtype not in DT_CODE or x.shape[1] != (num_heads + num_kv_heads) * head_dim + num_kv_heads * value_dim or positions.numel() != n
            or tuple(q_out.shape) != (n, num_heads * D) or rotary_dim % 2 or rotary_dim > head_dim):
        raise KernelError("rotary_unit_store: shapes do not agree")
    if rotary_dim:
        _need(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("rotary_unit_store: inv_freq must have rotary_dim / 2 entries")
    write = slots is not None
    if write:
        _need(slots, "slots", torch.int32), _need(k_pool, "k_pool", x.dtype), _need(v_pool, "v_pool", x.dtype)
        if tuple(k_pool.shape[1:]) != (num_kv_heads, page_size, D) or k_pool.shape != v_pool.shape or slots.numel() != n:
            raise KernelError("rotary_unit_store: pool layout must be [pages, kv_heads, page_size, max(head_dim, value_dim)]")
    f = _fn("attention_prep.cu", "dli_rotary_unit_store",
            [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 6 + [c_float, c_int, c_int, c_void_p])
    _check(f(_ptr(q_out), _ptr(x), x.stride(0), _ptr(positions), _ptr(inv_freq if rotary_dim else None), _ptr(slots if write else None),
             _ptr(k_pool if write else None), _ptr(v_pool if write else None), n, num_heads, num_kv_heads, head_dim, value_dim, rotary_dim,
             -1.0 if unit_eps is None else float(unit_eps), page_size, DT_CODE[x.dtype], _stream()), "rotary_unit_store")


def heads_matvec_supported(in_features: int, features: int) -> bool:
    """Sizes the small per-head product takes: a CTA of 256 threads covers the features (eight a thread when they are a
    multiple of 8), and the token's inputs and the partial sums fit 48 KB of shared memory."""
    runs = features // 8 if features % 8 == 0 and features // 8 <= 256 else features
    if runs > 256:
        return False
    slices = min(256 // runs, in_features)
    return (in_features + slices * features) * 4 <= 48 * 1024


def heads_matvec(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor | None = None) -> None:
    """out[t, h, :] = x[t, h, :] @ weight[h] (float32 sums), times sigmoid(gate[t, h, :]) if given: a product per head for a
    decode step's few tokens.  x [n, heads, in] and out [n, heads, features] may be column slices of wider rows (unit
    stride along the last axis); weight [heads, in, features] contiguous; gate [n, heads * features], a column slice too."""
    n, heads, feat = out.shape
    if (x.dtype not in DT_CODE or out.dtype != x.dtype or weight.dtype != x.dtype or not (x.is_cuda and out.is_cuda and weight.is_cuda)
            or x.shape[:2] != (n, heads) or tuple(weight.shape) != (heads, x.shape[2], feat) or not weight.is_contiguous()
            or x.stride(2) != 1 or out.stride(2) != 1):
        raise KernelError("heads_matvec: shapes, strides or dtypes do not agree")
    gate_row = 0
    if gate is not None:
        if gate.dtype != x.dtype or tuple(gate.shape) != (n, heads * feat) or gate.stride(1) != 1 or not gate.is_cuda:
            raise KernelError("heads_matvec: the gate must be [n, heads * features] with unit column stride")
        gate_row = gate.stride(0)
    f = _fn("attention_prep.cu", "dli_heads_matvec", [c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_longlong]
            + [c_int] * 5 + [c_void_p])
    _check(f(c_void_p(out.data_ptr()), out.stride(0), out.stride(1), c_void_p(x.data_ptr()), x.stride(0), x.stride(1), _ptr(weight),
             c_void_p(gate.data_ptr() if gate is not None else 0), gate_row, n, heads, x.shape[2], feat, DT_CODE[x.dtype], _stream()), "heads_matvec")


# ------------------------------------------------------------------ state-space mixer


def _columns(u: torch.Tensor, name: str) -> None:
    if u.dtype not in DT_CODE or u.dim() != 2 or not u.is_cuda or not u.is_contiguous():
        raise KernelError(f"{name}: the projection must be a contiguous CUDA matrix")


def causal_conv_silu(out: torch.Tensor, u: torch.Tensor, col0: int, weight: torch.Tensor, bias: torch.Tensor | None, state: torch.Tensor,
                     seq_of_token: torch.Tensor, q_start: torch.Tensor, state_slot: torch.Tensor, activation: bool = True) -> None:
    """out[t, c] = silu(bias[c] + sum_j weight[j, c] * in(t - (taps - 1) + j, c)) for channels c = columns col0 .. of u
    (``weight`` [taps, C]: each tap's weights lie together); with ``activation`` false the sum itself, without SiLU.
    The last tap weighs the token itself; in() before the step's first token of a sequence is the sequence's carried
    input in ``state`` [slots, taps - 1, C] (oldest first).  ``conv_state_update`` moves the state on afterwards."""
    _columns(u, "causal_conv_silu"), _need(out, "out", u.dtype), _need(weight, "weight", torch.float32), _need(state, "state", u.dtype)
    _need(seq_of_token, "seq_of_token", torch.int32), _need(q_start, "q_start", torch.int32), _need(state_slot, "state_slot", torch.int32)
    n, C = out.shape
    taps = weight.shape[0]
    if u.shape[0] != n or col0 + C > u.shape[1] or weight.shape[1] != C or tuple(state.shape[1:]) != (taps - 1, C) or seq_of_token.numel() != n:
        raise KernelError("causal_conv_silu: shapes do not agree")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    f = _fn("ssm.cu", "dli_causal_conv_silu", [c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(u), u.stride(0), col0, _ptr(weight), _ptr(bias), _ptr(state), _ptr(seq_of_token), _ptr(q_start), _ptr(state_slot),
             n, C, taps, int(activation), DT_CODE[u.dtype], _stream()), "causal_conv_silu")


def conv_state_update(state: torch.Tensor, u: torch.Tensor, col0: int, q_start: torch.Tensor, state_slot: torch.Tensor) -> None:
    """Each sequence's carried inputs ``state`` [slots, taps - 1, C] become the last taps - 1 inputs it has seen."""
    _columns(u, "conv_state_update"), _need(state, "state", u.dtype), _need(q_start, "q_start", torch.int32), _need(state_slot, "state_slot", torch.int32)
    _, keep, C = state.shape
    if col0 + C > u.shape[1] or q_start.numel() != state_slot.numel() + 1:
        raise KernelError("conv_state_update: shapes do not agree")
    f = _fn("ssm.cu", "dli_conv_state_update", [c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(state), _ptr(u), u.stride(0), col0, _ptr(q_start), _ptr(state_slot), state_slot.numel(), C, keep + 1, DT_CODE[u.dtype], _stream()),
           "conv_state_update")


SSM_SCAN_MAX_STATE = 512


def ssm_scan(y: torch.Tensor, xbc: torch.Tensor, u: torch.Tensor, dt_col: int, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
             state: torch.Tensor, q_start: torch.Tensor, state_slot: torch.Tensor, groups: int, max_len: int = 1 << 30) -> None:
    """The selective scan of every sequence's tokens of this step, from and to its slot of ``state`` [slots, heads, P, N]
    (float32; S transposed, so that a column's N values are contiguous).  xbc [n, heads P + 2 groups N] holds x | B | C; dt_raw is column dt_col + head of u.  Per head:
    dt = softplus(dt_raw + dt_bias), S <- exp(-exp(a_log) dt) S + dt B x^T, y = S^T C + d_skip x.  y [n, heads P] float32.
    ``max_len``: the most tokens a sequence brings, if the host knows (a launch hint: nothing is fetched ahead for single tokens)."""
    _columns(u, "ssm_scan"), _need(xbc, "xbc", u.dtype), _need(y, "y", torch.float32), _need(state, "state", torch.float32)
    for t, name in ((dt_bias, "dt_bias"), (a_log, "a_log"), (d_skip, "d_skip")):
        _need(t, name, torch.float32)
    _need(q_start, "q_start", torch.int32), _need(state_slot, "state_slot", torch.int32)
    _, heads, P, N = state.shape
    n = xbc.shape[0]
    if (xbc.shape[1] != heads * P + 2 * groups * N or tuple(y.shape) != (n, heads * P) or u.shape[0] != n or dt_col + heads > u.shape[1]
            or heads % groups or N > SSM_SCAN_MAX_STATE or dt_bias.numel() != heads or a_log.numel() != heads or d_skip.numel() != heads
            or q_start.numel() != state_slot.numel() + 1):
        raise KernelError(f"ssm_scan: shapes do not agree (or the state size is above {SSM_SCAN_MAX_STATE})")
    f = _fn("ssm.cu", "dli_ssm_scan", [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
            + [c_int] * 7 + [c_void_p])
    _check(f(_ptr(y), _ptr(xbc), _ptr(u), u.stride(0), dt_col, _ptr(dt_bias), _ptr(a_log), _ptr(d_skip), _ptr(state), _ptr(q_start),
             _ptr(state_slot), state_slot.numel(), heads, P, N, groups, int(max_len), DT_CODE[u.dtype], _stream()), "ssm_scan")


def gated_group_rmsnorm(out: torch.Tensor, y: torch.Tensor, u: torch.Tensor, z_col: int, weight: torch.Tensor, parts: int, eps: float,
                        gate_after: bool = False, gate: str = "silu") -> None:
    """out = g / sqrt(mean(g^2) + eps) * weight with g = y * silu(z), the mean taken over each of ``parts`` equal runs
    of the row; z is columns z_col .. of u; y float32.  ``gate_after``: the gate stays out of the norm,
    out = y / sqrt(mean(y^2) + eps) * weight * silu(z); with ``gate`` = ``"sigmoid"`` (only behind the norm) the gate is
    the logistic function of z instead of SiLU."""
    if gate not in ("silu", "sigmoid") or (gate == "sigmoid" and not gate_after):
        raise KernelError("gated_group_rmsnorm: gate is silu, or sigmoid behind the norm")
    _columns(u, "gated_group_rmsnorm"), _need(out, "out", u.dtype), _need(y, "y", torch.float32), _need(weight, "weight", torch.float32)
    n, inner = y.shape
    if tuple(out.shape) != (n, inner) or u.shape[0] != n or z_col + inner > u.shape[1] or weight.numel() != inner or inner % parts:
        raise KernelError("gated_group_rmsnorm: shapes do not agree")
    f = _fn("ssm.cu", "dli_gated_group_rmsnorm", [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p])
    mode = 2 if gate == "sigmoid" else int(gate_after)
    _check(f(_ptr(out), _ptr(y), _ptr(u), u.stride(0), z_col, _ptr(weight), n, inner, parts, eps, mode, DT_CODE[u.dtype], _stream()),
           "gated_group_rmsnorm")


# ------------------------------------------------------------------ gated delta rule

DELTA_MAX_HEAD_DIM = 512


def delta_rule_scan(o: torch.Tensor, qkv: torch.Tensor, u: torch.Tensor, b_col: int, a_col: int, dt_bias: torch.Tensor, a_log: torch.Tensor,
                    state: torch.Tensor, seq_of_token: torch.Tensor, q_start: torch.Tensor, state_slot: torch.Tensor, kv_heads: int, head_dim: int,
                    unit_eps: float, max_len: int = 1 << 30) -> None:
    """The gated delta rule over every sequence's tokens of this step, from and to its slot of ``state``
    [slots, heads, dv, d] (float32; S transposed, so that a value column's d numbers are contiguous).
    qkv [n, 2 kv_heads d + heads dv] holds q | k | v after convolution and activation; b and a are columns b_col + head and
    a_col + head of u.  Per head h (q/k head h // (heads / kv_heads)): q and k are divided by sqrt(sum of squares + unit_eps),
    q also by sqrt(d); beta = sigmoid(b), gamma = exp(-exp(a_log) softplus(a + dt_bias));
    S <- gamma S, w = beta (v - S^T k), S <- S + k w^T, o = S^T q.  o [n, heads dv] float32."""
    _columns(u, "delta_rule_scan"), _need(qkv, "qkv", u.dtype), _need(o, "o", torch.float32), _need(state, "state", torch.float32)
    _need(dt_bias, "dt_bias", torch.float32), _need(a_log, "a_log", torch.float32)
    _need(seq_of_token, "seq_of_token", torch.int32), _need(q_start, "q_start", torch.int32), _need(state_slot, "state_slot", torch.int32)
    _, heads, dv, d = state.shape
    n = qkv.shape[0]
    if (d != head_dim or kv_heads < 1 or heads % kv_heads or qkv.shape[1] != 2 * kv_heads * d + heads * dv or tuple(o.shape) != (n, heads * dv)
            or u.shape[0] != n or b_col + heads > u.shape[1] or a_col + heads > u.shape[1] or d > DELTA_MAX_HEAD_DIM or seq_of_token.numel() != n
            or dt_bias.numel() != heads or a_log.numel() != heads or q_start.numel() != state_slot.numel() + 1):
        raise KernelError(f"delta_rule_scan: shapes do not agree (or the head size is above {DELTA_MAX_HEAD_DIM})")
    # the float32 rows the recurrence reads, written by the first two of the three kernels: unit vectors, values, four numbers a
    # head, and every token's coefficients with the tokens of its tile of 16 (csrc/delta_rule.cu: row_layout)
    stride = ((2 * kv_heads * d + heads * dv + 3) & ~3) + 4 * heads + 2 * heads * 16
    scratch = torch.empty(n * stride, dtype=torch.float32, device=o.device)
    f = _fn("delta_rule.cu", "dli_delta_rule_scan", [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                                     c_void_p, c_void_p, c_void_p] + [c_int] * 7 + [c_float, c_int, c_void_p])
    _check(f(_ptr(o), _ptr(qkv), _ptr(u), u.stride(0), b_col, a_col, _ptr(dt_bias), _ptr(a_log), _ptr(state), _ptr(seq_of_token), _ptr(q_start),
             _ptr(state_slot), _ptr(scratch), n, state_slot.numel(), heads, kv_heads, d, dv, int(max_len), unit_eps, DT_CODE[u.dtype], _stream()),
           "delta_rule_scan")
    global launch_count
    launch_count += 2 if (max_len > 4 and d % 4 == 0 and dv % 4 == 0) else 1  # three kernels for portions, two for a decode step


# ------------------------------------------------------------------ a stream whose sublayers are normed on their output


def pair_embedding(h: torch.Tensor, table: torch.Tensor, scale: float, pair_table: torch.Tensor | None, buckets: int, mul_prev: int, mul_cur: int,
                   ids: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor, q_start: torch.Tensor, state_slot: torch.Tensor,
                   prev_state: torch.Tensor | None, y: torch.Tensor | None = None) -> None:
    """h[t] = table[ids[t]] * scale + pair_table[row(t)], float32.  row(t) = (prev * mul_prev + ids[t] * mul_cur) mod buckets, prev
    the token in front of t in its sequence; row ``buckets`` (the table's last) for a token at position 0.  The token in front of
    a sequence's first row of this step is prev_state[state_slot[s]] (int32 [slots]), where the step's last token is left for
    the next step.  Without ``pair_table`` only the first term.  With ``y`` (the tables' dtype) h is also written there, rounded once."""
    _need(h, "h", torch.float32), _need(table, "table"), _need(ids, "ids", torch.int32)
    n, H = h.shape
    if table.shape[1] != H or ids.numel() != n or table.dtype not in DT_CODE:
        raise KernelError("pair_embedding: shapes or dtype do not agree")
    if pair_table is not None:
        _need(pair_table, "pair_table", table.dtype), _need(prev_state, "prev_state", torch.int32)
        if tuple(pair_table.shape) != (buckets + 1, H):
            raise KernelError("pair_embedding: the pair table has buckets + 1 rows")
    f = _fn("residual_ops.cu", "dli_pair_embedding", [c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                      c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    if y is not None and (y.dtype != table.dtype or y.shape != h.shape or not y.is_contiguous()):
        raise KernelError("pair_embedding: y has h's shape and the tables' dtype")
    _check(f(_ptr(h), _ptr(table), float(scale), _ptr(pair_table), int(buckets), int(mul_prev), int(mul_cur), _ptr(ids), _ptr(positions),
             _ptr(seq_of_token), _ptr(q_start), _ptr(state_slot), _ptr(prev_state), _ptr(y), n, H, DT_CODE[table.dtype], _stream()), "pair_embedding")


def group_norm_add(h: torch.Tensor, a: torch.Tensor, weight: torch.Tensor, groups: int, eps: float, mult: float,
                   y: torch.Tensor | None = None) -> None:
    """h += mult * norm(a) * weight, norm = each of ``groups`` equal consecutive parts of a row divided by its own root mean
    square (eps inside the root); float32.  With ``y`` (a's dtype) the new h is also written there, rounded once."""
    _need(h, "h", torch.float32), _need(a, "a"), _need(weight, "weight", torch.float32)
    n, H = h.shape
    if tuple(a.shape) != (n, H) or weight.numel() != H or a.dtype not in DT_CODE or H % groups or (y is not None and (y.dtype != a.dtype or y.shape != a.shape)):
        raise KernelError("group_norm_add: shapes or dtype do not agree")
    if y is not None:
        _need(y, "y")
    f = _fn("residual_ops.cu", "dli_group_norm_add", [c_void_p, c_void_p, c_void_p, c_int, c_float, c_float, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(h), _ptr(a), _ptr(weight), int(groups), float(eps), float(mult), _ptr(y), n, H, DT_CODE[a.dtype], _stream()), "group_norm_add")


def group_norm_rows(y: torch.Tensor, h: torch.Tensor, weight: torch.Tensor, groups: int, eps: float, rows: torch.Tensor | None = None) -> None:
    """y[i] = norm(h[rows[i]]) * weight (rows None: every row), the norm of ``group_norm_add``."""
    _need(y, "y"), _need(h, "h", torch.float32), _need(weight, "weight", torch.float32)
    n, H = y.shape
    if h.shape[1] != H or y.dtype not in DT_CODE or H % groups or (rows is None and h.shape[0] != n) or (rows is not None and rows.numel() != n):
        raise KernelError("group_norm_rows: shapes or dtype do not agree")
    if rows is not None:
        _need(rows, "rows", torch.int32)
    f = _fn("residual_ops.cu", "dli_group_norm_rows", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(y), _ptr(h), _ptr(weight), _ptr(rows), int(groups), float(eps), n, H, DT_CODE[y.dtype], _stream()), "group_norm_rows")


def gelu_mul_rows(g: torch.Tensor, table: torch.Tensor, col0: int, ids: torch.Tensor) -> None:
    """g[t, j] = gelu_tanh(g[t, j]) * table[ids[t], col0 + j], in place (float32 arithmetic)."""
    _need(g, "g"), _need(table, "table", g.dtype), _need(ids, "ids", torch.int32)
    n, dim = g.shape
    if g.dtype not in DT_CODE or ids.numel() != n or col0 < 0 or col0 + dim > table.shape[1]:
        raise KernelError("gelu_mul_rows: shapes or dtype do not agree")
    f = _fn("residual_ops.cu", "dli_gelu_mul_rows", [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(g), _ptr(table), table.shape[1], int(col0), _ptr(ids), n, dim, DT_CODE[g.dtype], _stream()), "gelu_mul_rows")


def depth_average(out: torch.Tensor, x0: torch.Tensor, hist: torch.Tensor, weights: torch.Tensor, count: int, y: torch.Tensor | None = None) -> None:
    """out = weights[0] * x0 + sum over 1 <= j < count of weights[j] * hist[j - 1] (x0, out [n, H] and hist [slots, n, H] float32;
    out may be a slot of hist beyond the ones read).  With ``y`` the result is also written there in y's dtype."""
    _need(out, "out", torch.float32), _need(x0, "x0", torch.float32), _need(hist, "hist", torch.float32), _need(weights, "weights", torch.float32)
    if hist.dim() != 3 or tuple(hist.shape[1:]) != tuple(out.shape) or x0.shape != out.shape or not 1 <= count <= hist.shape[0] + 1 or weights.numel() < count:
        raise KernelError("depth_average: shapes do not agree")
    if y is not None:
        _need(y, "y")
        if y.dtype not in DT_CODE or y.shape != out.shape:
            raise KernelError("depth_average: y has out's shape")
    f = _fn("residual_ops.cu", "dli_depth_average", [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(x0), _ptr(hist), out.numel(), _ptr(weights), int(count), _ptr(y), out.numel(), DT_CODE[y.dtype] if y is not None else 0,
             _stream()), "depth_average")


MINGRU_CHUNK = 64  # rows of a sequence that one thread walks when a portion is cut into chunks


def mingru_scan(out: torch.Tensor, p: torch.Tensor, bz: torch.Tensor, bx: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor,
                state_slot: torch.Tensor, max_len: int = 0) -> None:
    """minGRU over any mix of prompt portions and single tokens.  p [n, 3 W] = z | x | g projections; per channel
    z = sigmoid(pz + bz), u = px + bx, c = u + 1/2 where u >= 0 else sigmoid(u), S <- (1 - z) S + z c, out = S * silu(pg).
    state [slots, W] float32 holds S per request; ``max_len``: the longest sequence's rows in this step (0: unknown, walk plainly)."""
    _need(out, "out"), _need(p, "p", out.dtype), _need(bz, "bz", torch.float32), _need(bx, "bx", torch.float32), _need(state, "state", torch.float32)
    n, W = out.shape
    seqs = state_slot.numel()
    if tuple(p.shape) != (n, 3 * W) or out.dtype not in DT_CODE or state.shape[1] != W or q_start.numel() != seqs + 1:
        raise KernelError("mingru_scan: shapes or dtype do not agree")
    scratch = None
    if max_len > 4 * MINGRU_CHUNK:
        cps = -(-max_len // MINGRU_CHUNK)
        scratch = torch.empty((2 * n + (2 * cps + 1) * seqs) * W, dtype=torch.float32, device=out.device)
    f = _fn("mingru.cu", "dli_mingru_scan", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                             c_int, c_void_p, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(p), _ptr(bz), _ptr(bx), _ptr(state), _ptr(q_start), _ptr(state_slot), n, seqs, W, int(max_len), MINGRU_CHUNK,
             _ptr(scratch), DT_CODE[out.dtype], _stream()), "mingru_scan")


def diff_prep(q_out: torch.Tensor, proj: torch.Tensor, k_col: int, v_col: int, wq: torch.Tensor, wk: torch.Tensor | None, eps: float,
              positions: torch.Tensor, freq: torch.Tensor, amp: float, slots: torch.Tensor | None, k_pool: torch.Tensor | None,
              v_pool: torch.Tensor | None, num_heads: int, num_kv_heads: int, dim: int, vdim: int, rot: int, page_size: int) -> None:
    """Query and key preparation of differential attention.  proj rows hold q [heads][2 maps][dim] from column 0 and, when the
    layer has keys and values of its own (k_col >= 0), k [kv_heads][2][dim] from k_col and v [kv_heads][vdim] from v_col.
    Every map of every head is divided by its root mean square over dim (eps inside the root) and multiplied by wq (wk), then
    its first ``rot`` dimensions are rotated in pairs (2i, 2i + 1) by the angle position * freq[i], cosine and sine times ``amp``.
    q goes to q_out [n, heads * 2 * dim]; k and v go to the pages at ``slots`` (k_pool [pages, kv_heads, page_size, 2 dim],
    v_pool [pages, kv_heads, page_size, vdim])."""
    _need(q_out, "q_out"), _need(proj, "proj", q_out.dtype), _need(wq, "wq", torch.float32), _need(freq, "freq", torch.float32)
    n = proj.shape[0]
    writes = k_col >= 0
    if q_out.dtype not in DT_CODE or tuple(q_out.shape) != (n, num_heads * 2 * dim) or rot % 2 or rot > dim or freq.numel() < rot // 2:
        raise KernelError("diff_prep: shapes or dtype do not agree")
    if writes:
        _need(wk, "wk", torch.float32), _need(slots, "slots", torch.int32), _need(k_pool, "k_pool", q_out.dtype), _need(v_pool, "v_pool", q_out.dtype)
        if tuple(k_pool.shape[1:]) != (num_kv_heads, page_size, 2 * dim) or tuple(v_pool.shape[1:]) != (num_kv_heads, page_size, vdim):
            raise KernelError("diff_prep: the pools' shapes do not agree with the heads")
    f = _fn("diff_attention.cu", "dli_diff_prep", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_float,
                                                   c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(q_out), _ptr(proj), proj.shape[1], int(k_col), int(v_col), _ptr(wq), _ptr(wk), float(eps), _ptr(positions), _ptr(freq), float(amp),
             _ptr(slots if writes else None), _ptr(k_pool if writes else None), _ptr(v_pool if writes else None), n, num_heads, num_kv_heads, dim,
             vdim, rot, page_size, DT_CODE[q_out.dtype], _stream()), "diff_prep")


def diff_attention_simt(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_tables: torch.Tensor,
                        seq_of_token: torch.Tensor, positions: torch.Tensor, gate: torch.Tensor | None, num_heads: int, scale: float,
                        window: int | None, keep_first: int, lam: float, post: float, eps: float) -> None:
    """Differential attention on CUDA cores for every token of the step, both maps, the difference a1 - lam * a2, the head's
    RMS norm (no weight) times ``post`` and the gate sigmoid(gate[t, head]) in one kernel.  q [n, heads * 2 * dim] (prepared),
    out [n, heads * vdim]; ``gate`` [n, heads] may be a column slice of wider rows (or None).  Position i sees j <= i when
    i - j < window or j < keep_first (window None: all)."""
    _need(out, "out"), _need(q, "q", out.dtype), _need(k_pool, "k_pool", out.dtype), _need(v_pool, "v_pool", out.dtype)
    n = q.shape[0]
    _, nkv, page_size, d2 = k_pool.shape
    vdim = v_pool.shape[3]
    if out.dtype not in DT_CODE or d2 % 2 or tuple(q.shape) != (n, num_heads * d2) or tuple(out.shape) != (n, num_heads * vdim) or num_heads % nkv:
        raise KernelError("diff_attention_simt: shapes or dtype do not agree")
    gate_stride = 0
    if gate is not None:
        if gate.dtype != out.dtype or gate.shape != (n, num_heads) or gate.stride(1) != 1 or not gate.is_cuda:
            raise KernelError("diff_attention_simt: gate must be [n, heads] with unit column stride")
        gate_stride = gate.stride(0)
    f = _fn("diff_attention.cu", "dli_diff_attention_simt", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                                             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                                             c_float, c_float, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_tables), block_tables.shape[1], _ptr(seq_of_token), _ptr(positions),
             _ptr(gate), gate_stride, n, num_heads, nkv, d2 // 2, vdim, page_size, int(window or 0), int(keep_first), float(scale), float(lam),
             float(post), float(eps), DT_CODE[out.dtype], _stream()), "diff_attention_simt")


def _diff_attention_tc_smem(dim: int, vdim: int) -> int:
    stages = 64 * (8 * dim + 4 * vdim + 64)  # two stages of 64 key and value rows; the warps' partial results take their place at the end
    partial = 512 * (vdim + (8 if vdim % 32 == 0 else 24))
    return 64 * (4 * dim + 16) + max(stages, partial)  # and 64 query rows in front of them


def diff_attention_tc_supported(dim: int, vdim: int) -> bool:
    """Sizes of a map's keys and of the values that the tensor-core kernel of differential attention takes (bfloat16)."""
    return dim % 16 == 0 and vdim % 16 == 0 and 16 <= dim <= 256 and 16 <= vdim <= 256 and _diff_attention_tc_smem(dim, vdim) <= 227 * 1024


def diff_attention_tc_ctas_per_sm(dim: int, vdim: int) -> int:
    """CTAs of the tensor-core kernel that an SM holds at once (the kernel's own rule: two where 128 registers a thread and
    half the shared memory suffice)."""
    return 2 if dim <= 128 and vdim <= 128 and 2 * _diff_attention_tc_smem(dim, vdim) + 2048 <= 227 * 1024 else 1


def diff_attention_tc(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_tables: torch.Tensor,
                      q_start: torch.Tensor, kv_len: torch.Tensor, num_seqs: int, max_q_len: int, gate: torch.Tensor | None, num_heads: int,
                      scale: float, window: int | None, keep_first: int, lam: float, post: float, eps: float, splits: int = 1,
                      scratch: torch.Tensor | None = None) -> None:
    """``diff_attention_simt`` on tensor cores (bfloat16; one library per pair of sizes): sequences given by their first rows
    ``q_start`` [seqs + 1] and lengths in the cache after this step ``kv_len`` [seqs]; prompt portions and single tokens in one
    launch, sized for ``max_q_len`` rows a sequence.  ``splits`` > 1 (single tokens only): the key tiles of every sequence are
    divided between that many CTAs, whose partial results meet in ``scratch`` (float32, ``diff_attention_scratch`` numbers)
    and are merged by a second kernel."""
    _need(out, "out", torch.bfloat16), _need(q, "q", torch.bfloat16), _need(k_pool, "k_pool", torch.bfloat16), _need(v_pool, "v_pool", torch.bfloat16)
    n = q.shape[0]
    _, nkv, page_size, d2 = k_pool.shape
    vdim = v_pool.shape[3]
    if not diff_attention_tc_supported(d2 // 2, vdim) or tuple(q.shape) != (n, num_heads * d2) or tuple(out.shape) != (n, num_heads * vdim) or num_heads % nkv:
        raise KernelError("diff_attention_tc: shapes do not agree or sizes not supported")
    gate_stride = 0
    if gate is not None:
        if gate.dtype != out.dtype or gate.shape != (n, num_heads) or gate.stride(1) != 1 or not gate.is_cuda:
            raise KernelError("diff_attention_tc: gate must be [n, heads] with unit column stride")
        gate_stride = gate.stride(0)
    splits = max(1, int(splits))
    if splits > 1:
        if max_q_len != 1:
            raise KernelError("diff_attention_tc: keys are split between CTAs for single tokens only")
        need = diff_attention_scratch(num_seqs, num_heads, vdim, splits)
        if scratch is None or scratch.dtype != torch.float32 or not scratch.is_contiguous() or scratch.numel() < need or scratch.device != out.device:
            raise KernelError(f"diff_attention_tc: {splits} splits need a float32 scratch of {need} numbers")
    f = _fn("diff_attention.cu", "dli_diff_attention_tc", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                                           c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_float,
                                                           c_int, c_void_p, c_void_p], defines={"DIFF_DK": d2 // 2, "DIFF_DV": vdim})
    _check(f(_ptr(out), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_tables), block_tables.shape[1], _ptr(q_start), _ptr(kv_len), int(num_seqs),
             int(max_q_len), _ptr(gate), gate_stride, num_heads, nkv, page_size, int(window or 0), int(keep_first), float(scale), float(lam),
             float(post), float(eps), splits, _ptr(scratch) if splits > 1 else None, _stream()), "diff_attention_tc")


def diff_attention_scratch(num_seqs: int, num_heads: int, vdim: int, splits: int) -> int:
    """float32 numbers of the scratch in which ``splits`` CTAs leave a single token's partial results: for every sequence,
    head, split and map the unnormalised outputs, their maximum and their sum."""
    return num_seqs * num_heads * splits * 2 * (vdim + 2)


# ------------------------------------------------------------------ a stream whose sublayer outputs carry a learned scale per feature


def add_rmsnorm_scaled(y: torch.Tensor | None, h: torch.Tensor, a: torch.Tensor | None, fa: float, b: torch.Tensor | None, fb: float,
                       scale: torch.Tensor | None, weight: torch.Tensor | None, eps: float, rows: torch.Tensor | None = None) -> None:
    """v = h[s] + scale * (fa * a[s] + fb * b[s]) with s = rows[r] (or r); y[r] = v / sqrt(mean(v^2) + eps) * weight.
    ``b`` may be None (one output), ``a`` too (nothing is added).  Without ``rows`` the sum is written back to ``h``; with
    ``y`` None only the addition happens.  float32 arithmetic, one rounding."""
    _need(h, "h", torch.float32)
    H = h.shape[1]
    n_rows = h.shape[0] if rows is None else rows.numel()
    dtype = y.dtype if y is not None else (a.dtype if a is not None else torch.float32)
    if dtype not in DT_CODE:
        raise KernelError("add_rmsnorm_scaled: dtype not supported")
    if y is not None:
        _need(y, "y", dtype), _need(weight, "weight", torch.float32)
        if tuple(y.shape) != (n_rows, H) or weight.numel() != H:
            raise KernelError("add_rmsnorm_scaled: y or weight has the wrong shape")
    for t, name in ((a, "a"), (b, "b")):
        if t is not None:
            _need(t, name, dtype)
            if t.shape != h.shape:
                raise KernelError(f"add_rmsnorm_scaled: {name} must have the stream's shape")
    if a is not None:
        _need(scale, "scale", torch.float32)
        if scale.numel() != H:
            raise KernelError("add_rmsnorm_scaled: one scale per feature")
    if b is not None and a is None:
        raise KernelError("add_rmsnorm_scaled: b without a")
    if rows is not None:
        _need(rows, "rows", torch.int32)
    if y is None and (rows is not None or a is None):
        return
    f = _fn("stream_ops.cu", "dli_add_rmsnorm_scaled", [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_float, c_void_p, c_void_p, c_float, c_void_p,
                                                        c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(y), _ptr(h), _ptr(a), float(fa), _ptr(b), float(fb), _ptr(scale), _ptr(weight), eps, _ptr(rows), n_rows, H, DT_CODE[dtype], _stream()),
           "add_rmsnorm_scaled")


def concat_stream_rows(out: torch.Tensor, h: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> None:
    """out[t] = [h[t] rounded to out's dtype | table[ids[t]]]: the stream and the embedding of the step's tokens side by side."""
    _need(out, "out"), _need(h, "h", torch.float32), _need(table, "table", out.dtype), _need(ids, "ids", torch.int32)
    n, W = h.shape
    if out.dtype not in DT_CODE or tuple(out.shape) != (n, 2 * W) or table.shape[1] != W or ids.numel() != n:
        raise KernelError("concat_stream_rows: shapes or dtype do not agree")
    f = _fn("stream_ops.cu", "dli_concat_stream_rows", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(h), _ptr(table), _ptr(ids), n, W, DT_CODE[out.dtype], _stream()), "concat_stream_rows")


def token_shift_blend(out: torch.Tensor, x: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, seq_of_token: torch.Tensor, q_start: torch.Tensor,
                      state_slot: torch.Tensor) -> None:
    """out[j, t] = x[t] + (before(t) - x[t]) * mu[j]: ``mu`` [blends, W] float32; before(t) is the row of the token in front of t in its
    sequence — x[t - 1] inside the step, the sequence's carried row ``state`` [slots, 1, W] at the step's first token.
    ``conv_state_update`` (one carried row) moves the state on afterwards."""
    _need(out, "out"), _need(x, "x", out.dtype), _need(mu, "mu", torch.float32), _need(state, "state", out.dtype)
    _need(seq_of_token, "seq_of_token", torch.int32), _need(q_start, "q_start", torch.int32), _need(state_slot, "state_slot", torch.int32)
    n, W = x.shape
    blends = mu.shape[0]
    if out.dtype not in DT_CODE or tuple(out.shape) != (blends, n, W) or mu.shape[1] != W or tuple(state.shape[1:]) != (1, W) or seq_of_token.numel() != n:
        raise KernelError("token_shift_blend: shapes or dtype do not agree")
    f = _fn("stream_ops.cu", "dli_token_shift_blend", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(x), _ptr(mu), _ptr(state), _ptr(seq_of_token), _ptr(q_start), _ptr(state_slot), n, W, blends, DT_CODE[out.dtype], _stream()),
           "token_shift_blend")


# ------------------------------------------------------------------ recurrences whose state decays per head and key channel

RECURRENCE_MAX_HEAD_DIM = 512


def decay_recurrence_row(kq_heads: int, heads: int, d: int, dv: int) -> int:
    """Floats of a token's row as ``decay_recurrence`` reads it: A [kq_heads, d] (what the state is read with) | K [kq_heads, d] |
    G [heads, d] (decays) | V [heads, dv] | B [heads] (betas), rounded up to a multiple of 4 (csrc/recurrence.cu: row_layout)."""
    return (2 * kq_heads * d + heads * d + heads * dv + heads + 3) & ~3


def shift_decay_prep(rows: torch.Tensor, rkvg: torch.Tensor, wz: torch.Tensor, w0: torch.Tensor, heads: int, d: int) -> None:
    """The float32 rows of the token-shift recurrence: A = r, K = k, V = v (slabs 0, 1, 2 of ``rkvg`` [4, n, heads d]) and the decays
    G = exp(-exp(wz + w0)) (``wz`` [n, heads d], ``w0`` [heads d] float32)."""
    _need(rows, "rows", torch.float32), _need(rkvg, "rkvg"), _need(wz, "wz", rkvg.dtype), _need(w0, "w0", torch.float32)
    n, I = wz.shape
    if rkvg.dtype not in DT_CODE or I != heads * d or tuple(rkvg.shape) != (4, n, I) or w0.numel() != I or tuple(rows.shape) != (n, decay_recurrence_row(heads, heads, d, d)):
        raise KernelError("shift_decay_prep: shapes or dtype do not agree")
    f = _fn("recurrence.cu", "dli_shift_decay_prep", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(rows), _ptr(rkvg), _ptr(wz), _ptr(w0), n, heads, d, DT_CODE[rkvg.dtype], _stream()), "shift_decay_prep")


def channel_delta_prep(rows: torch.Tensor, qkv: torch.Tensor, u: torch.Tensor, b_col: int, a: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor,
                       heads: int, kv_heads: int, d: int, dv: int, unit_eps: float) -> None:
    """The float32 rows of the delta rule with a decay per channel.  qkv [n, 2 kv_heads d + heads dv]: q | k | v after convolution and
    activation; q and k become unit vectors per head (``unit_eps`` inside the root), q also times d^-1/2; B = sigmoid(u[:, b_col + h]);
    G = exp(-exp(a_log[h]) softplus(a[:, h d + i] + dt_bias[h d + i]))."""
    _columns(u, "channel_delta_prep"), _need(rows, "rows", torch.float32), _need(qkv, "qkv", u.dtype), _need(a, "a", u.dtype)
    _need(dt_bias, "dt_bias", torch.float32), _need(a_log, "a_log", torch.float32)
    n = qkv.shape[0]
    if (kv_heads < 1 or heads % kv_heads or qkv.shape[1] != 2 * kv_heads * d + heads * dv or tuple(a.shape) != (n, heads * d) or u.shape[0] != n
            or b_col + heads > u.shape[1] or dt_bias.numel() != heads * d or a_log.numel() != heads
            or tuple(rows.shape) != (n, decay_recurrence_row(kv_heads, heads, d, dv))):
        raise KernelError("channel_delta_prep: shapes do not agree")
    f = _fn("recurrence.cu", "dli_channel_delta_prep", [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p] + [c_int] * 5
            + [c_float, c_int, c_void_p])
    _check(f(_ptr(rows), _ptr(qkv), _ptr(u), u.stride(0), b_col, _ptr(a), _ptr(dt_bias), _ptr(a_log), n, heads, kv_heads, d, dv, unit_eps,
             DT_CODE[u.dtype], _stream()), "channel_delta_prep")


def decay_recurrence(o: torch.Tensor, rows: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor, state_slot: torch.Tensor, kq_heads: int,
                     mode: str, bonus: torch.Tensor | None = None, max_len: int = 1 << 30, rows_per_lane: int = 0) -> None:
    """A linear recurrence over every sequence's tokens of this step, from and to its slot of ``state`` [slots, heads, dv, d] (float32; S
    transposed, so that a value column's d numbers are contiguous).  ``rows`` [n, decay_recurrence_row(...)] float32.  Per head, with
    a, k (of q/k head h // (heads / kq_heads)), decays g [d], values v [dv]:

    ``"bonus"``:  o = (S + diag(u) k v^T)^T a;   S <- diag(g) S + k v^T          (``bonus`` [heads, d]: u)
    ``"delta"``:  S <- diag(g) S;   w = beta (v - S^T k);   S <- S + k w^T;   o = S^T a

    o [n, heads dv] float32.  Tokens are walked in order.  ``rows_per_lane`` (32, 16, 8; 0: the launcher chooses from the step's shape):
    how many key rows of a column one lane keeps, which fixes the order in which the sums over d are added."""
    _need(o, "o", torch.float32), _need(rows, "rows", torch.float32), _need(state, "state", torch.float32)
    _need(q_start, "q_start", torch.int32), _need(state_slot, "state_slot", torch.int32)
    _, heads, dv, d = state.shape
    n = rows.shape[0]
    if mode not in ("bonus", "delta") or (mode == "bonus") != (bonus is not None):
        raise KernelError("decay_recurrence: mode is bonus (with its vector) or delta")
    if bonus is not None:
        _need(bonus, "bonus", torch.float32)
        if tuple(bonus.shape) != (heads, d):
            raise KernelError("decay_recurrence: bonus must be [heads, d]")
    if (kq_heads < 1 or heads % kq_heads or d > RECURRENCE_MAX_HEAD_DIM or tuple(o.shape) != (n, heads * dv) or rows.shape[1] != decay_recurrence_row(kq_heads, heads, d, dv)
            or q_start.numel() != state_slot.numel() + 1):
        raise KernelError(f"decay_recurrence: shapes do not agree (or the head size is above {RECURRENCE_MAX_HEAD_DIM})")
    f = _fn("recurrence.cu", "dli_decay_recurrence", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 7 + [c_void_p])
    _check(f(_ptr(o), _ptr(rows), _ptr(state), _ptr(q_start), _ptr(state_slot), _ptr(bonus), state_slot.numel(), heads, kq_heads, d, dv,
             0 if mode == "bonus" else 1, int(rows_per_lane), _stream()), "decay_recurrence")


# ------------------------------------------------------------------ routed mixture of gated feed-forwards

MOE_MAX_TOP = 32
MOE_GROUPED_TILE_ROWS = 64  # BM of csrc/moe_grouped.cu
MOE_GROUPED_MIN_TOKENS = 4  # fewer tokens rarely share an expert: every chosen expert is read once per pair, on the CUDA cores


def moe_grouped_supported(tokens: int, W: int, ff: int, dtype: torch.dtype) -> bool:
    """Whether the experts' products of a step go to the grouped tensor-core kernels: bfloat16, more tokens than a decode step
    brings, rows of whole 16-byte chunks."""
    return dtype == torch.bfloat16 and tokens >= MOE_GROUPED_MIN_TOKENS and W % 8 == 0 and ff % 8 == 0
MOE_PAIR_CHUNK = 8192  # tokens a launch of the pair kernels takes (their grids count (token, expert) pairs along y)


def moe_route(ids: torch.Tensor, weights: torch.Tensor, x: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, group_count: int,
              group_keep: int, scale: float) -> None:
    """Which experts every token uses, and with what weights.  z = x router^T (float32), s = sigmoid(z), choice = s + correction.
    With ``group_count`` > 1 the experts form equal groups of neighbours, a group's mark is the sum of its two largest choice scores,
    and only experts of the ``group_keep`` best groups are eligible.  ids [n, top] int32: the eligible experts with the largest choice
    scores, best first (ties: the lower index); weights [n, top] float32 = s[ids] / (their sum + 1e-20) * scale."""
    _need(ids, "ids", torch.int32), _need(weights, "weights", torch.float32), _need(x, "x"), _need(router, "router", torch.float32)
    _need(correction, "correction", torch.float32)
    n, W = x.shape
    E, top = router.shape[0], ids.shape[1]
    if (x.dtype not in DT_CODE or router.shape[1] != W or correction.numel() != E or tuple(ids.shape) != (n, top) or tuple(weights.shape) != (n, top)
            or top > MOE_MAX_TOP or group_count < 1 or E % group_count or not 1 <= group_keep <= group_count or top > group_keep * (E // group_count)):
        raise KernelError("moe_route: shapes, dtype or groups do not agree")
    f = _fn("moe.cu", "dli_moe_route", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 6 + [c_float, c_int, c_void_p])
    _check(f(_ptr(ids), _ptr(weights), _ptr(x), _ptr(router), _ptr(correction), n, W, E, top, group_count, group_keep, float(scale), DT_CODE[x.dtype],
             _stream()), "moe_route")


def moe_experts(out: torch.Tensor, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor,
                activation: str = "silu", stages: int = 0) -> None:
    """out[t] = sum_k weights[t, k] * down_e(act(gate_e x[t]) * (up_e x[t])), e = ids[t, k], added in the order of k in float32.
    w_gate_up [E, 2 ff, W] (an expert's gate rows, then its up rows), w_down [E, W, ff].  The two inner sums are rounded to the
    activation dtype before the activation, and so is their product.  ``stages`` (2, 3; 0: chosen from the step's shape): how deep
    the grouped products' asynchronous copies run."""
    _need(out, "out"), _need(x, "x", out.dtype), _need(ids, "ids", torch.int32), _need(weights, "weights", torch.float32)
    _need(w_gate_up, "w_gate_up", out.dtype), _need(w_down, "w_down", out.dtype)
    n, W = x.shape
    top = ids.shape[1]
    E, ff2, _ = w_gate_up.shape
    ff = ff2 // 2
    if (out.dtype not in DT_CODE or tuple(out.shape) != (n, W) or w_gate_up.shape[2] != W or tuple(w_down.shape) != (E, W, ff) or tuple(ids.shape) != (n, top)
            or tuple(weights.shape) != (n, top) or activation not in GLU_ACTIVATIONS):
        raise KernelError("moe_experts: shapes, dtype or activation do not agree")
    global launch_count
    if moe_grouped_supported(n, W, ff, out.dtype):
        # many tokens: the pairs sorted by expert, two grouped products on the tensor cores (csrc/moe_grouped.cu)
        tiles = (min(n * top, E) + n * top // MOE_GROUPED_TILE_ROWS)
        rows = tiles * MOE_GROUPED_TILE_ROWS
        ints = torch.empty(2 * (E + 1) + 2 * n * top + tiles + rows, dtype=torch.int32, device=out.device)
        hidden = torch.empty((rows, ff), dtype=out.dtype, device=out.device)
        partial = torch.empty((rows, W), dtype=torch.float32, device=out.device)
        g = _fn("moe_grouped.cu", "dli_moe_grouped", [c_void_p] * 9 + [c_int] * 7 + [c_void_p])
        _check(g(_ptr(out), _ptr(x), _ptr(ids), _ptr(weights), _ptr(w_gate_up), _ptr(w_down), _ptr(ints), _ptr(hidden), _ptr(partial), n, W, ff, E, top,
                 GLU_ACTIVATIONS[activation], int(stages), _stream()), "moe_experts")
        launch_count += 3 if n * top <= 2048 else 6  # four kernels a call (one block sorts up to 2,048 pairs), else seven
        return
    f = _fn("moe.cu", "dli_moe_pairs", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 6 + [c_void_p])
    step = max(1, min(MOE_PAIR_CHUNK, 65535 // top))
    hidden = torch.empty((min(n, step) * top, ff), dtype=out.dtype, device=out.device)
    for t0 in range(0, n, step):
        m = min(step, n - t0)
        _check(f(_ptr(out[t0:]), _ptr(hidden), _ptr(x[t0:]), _ptr(ids[t0:]), _ptr(weights[t0:]), _ptr(w_gate_up), _ptr(w_down), m, W, ff, top,
                 GLU_ACTIVATIONS[activation], DT_CODE[out.dtype], _stream()), "moe_experts")
        launch_count += 1  # two kernels a call
