"""Tensor-level entry to the kernels: checks, then raw pointers and the current stream.

Every function writes into tensors that the caller provides; nothing here allocates.  All tensors must
be contiguous CUDA tensors.  Sizes a kernel cannot take are refused with a `KernelError` that says why;
no function has a CPU or library fallback.
"""
from __future__ import annotations

import os

import torch

from . import KernelError, call

F32, BF16 = 0, 1
ACT = {"none": 0, None: 0, "gelu_tanh": 1, "gelu_erf": 2, "relu2": 3}
#: gates of `gate_mul` (not taken by the products' epilogues)
GATE = {"silu": 4, "sigmoid": 5, "relu": 6, "gelu_tanh": 1}


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dt}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle.  Asked for at every launch, so by the short way where torch has one
    (`torch.cuda.current_stream()` builds a Stream object: about 5 us, a quarter of a launch's host time)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _dev(t: torch.Tensor, name: str, dtype=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must live on the CUDA device (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, not {t.dtype}")


def _rows(t: torch.Tensor, name: str, dtype=None) -> None:
    """A matrix whose rows may lie inside wider rows (a range of columns of a product's result): elements of a row
    contiguous, any row stride."""
    if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be a CUDA matrix whose rows are contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, not {t.dtype}")


def embed(wte, wpe, tokens, positions, out, dev_err, stats: "RowStats | None" = None) -> None:
    """out[t] = wte[tokens[t]] (+ wpe[positions[t]]), float32.  With `stats` and few rows (a decode step) the rows'
    statistics are left there for the next product's LayerNorm."""
    _dev(wte, "wte"); _dev(tokens, "tokens", torch.int32); _dev(out, "out", torch.float32)
    _dev(dev_err, "dev_err", torch.int32)
    T = tokens.shape[0]
    V, d = wte.shape
    P = 0
    if wpe is not None:
        _dev(wpe, "wpe", wte.dtype); _dev(positions, "positions", torch.int32)
        P = wpe.shape[0]
        if wpe.shape[1] != d or positions.shape[0] != T:
            raise KernelError("embed: position table or positions do not match")
    if out.shape[0] < T or out.shape[1] != d:
        raise KernelError("embed: output does not match")
    keep = stats is not None and stats.takes(T, d)     # few rows: a decode step; leave their statistics
    if stats is not None:
        stats.written(out)
    call("vlrf_embed", _ptr(wte), _ptr(wpe), dtype_code(wte.dtype), _ptr(tokens), _ptr(positions), _ptr(out),
         T, d, V, P, _ptr(stats.buffer()) if keep else 0, _ptr(dev_err), _stream())
    if keep:
        stats.keep(out, T, d)


def layernorm(x, gamma, beta, eps: float, out, rows=None) -> None:
    """out[r] = LN(x[rows[r]] if rows is given else x[r]); x float32, out float32 or bfloat16."""
    _dev(x, "x", torch.float32); _dev(gamma, "gamma", torch.float32); _dev(beta, "beta", torch.float32)
    _dev(out, "out")
    d = x.shape[1]
    n = x.shape[0]
    if rows is not None:
        _dev(rows, "rows", torch.int32)
        n = rows.shape[0]
    if gamma.shape[0] != d or beta.shape[0] != d or out.shape[1] != d or out.shape[0] < n:
        raise KernelError("layernorm: sizes do not match")
    call("vlrf_layernorm", _ptr(x), _ptr(rows), _ptr(gamma), _ptr(beta), _ptr(out), dtype_code(out.dtype), n, d,
         float(eps), _stream())


def linear(x, w, bias, out, *, act=None, residual=None, rows: int | None = None, kv_scatter=None,
           stats: "RowStats | None" = None) -> bool:
    """out = act(x · wᵀ + bias) (+ residual).  x [M,K], w [N,K] (same dtype), bias/residual float32,
    out [M,N] float32 or bfloat16.  `rows` limits M to the first rows of x/out/residual.  `kv_scatter`
    (see linear_layernorm) asks the kernel to write K/V columns into a cache as well; the return value
    says whether it did (only the tensor-core kernels can).  `stats`: where the statistics of float32 result rows
    are left when the kernel that takes the shape computes them (and where stale ones of `out` are forgotten)."""
    _dev(x, "x"); _dev(w, "w", x.dtype); _dev(out, "out")
    M = x.shape[0] if rows is None else rows
    K = x.shape[1]
    N = w.shape[0]
    if w.shape[1] != K or out.shape[1] != N or out.shape[0] < M or x.shape[0] < M:
        raise KernelError(f"linear: x {list(x.shape)}, w {list(w.shape)}, out {list(out.shape)} do not match")
    if bias is not None:
        _dev(bias, "bias", torch.float32)
        if bias.shape[0] != N:
            raise KernelError("linear: bias does not match")
    if residual is not None:
        _dev(residual, "residual", torch.float32)
        if residual.shape[1] != N or residual.shape[0] < M:
            raise KernelError("linear: residual does not match")
    if x.dtype == torch.float32 and out.dtype != torch.float32:
        raise KernelError("linear: float32 input gives float32 output")
    if stats is not None:
        stats.written(out)
    return _linear_dispatch(x, w, bias, out, ACT[act], residual, M, N, K, kv_scatter, stats)


#: head sizes that the attention kernels take (each checks it again; parts refuse others when they are built)
HEAD_DIM_STEP, HEAD_DIM_MAX = 16, 256
_SM_COUNT = None
USE_TCGEN05 = True
PREFILL_ATTENTION_TCGEN05 = True     # head size 64; off: the mma.sync kernel takes those too
PREFILL_ATTENTION_PARTS = None       # a number here overrides attention_prefill_parts (for measurements)
SKINNY_MAX_ROWS = 64
FUSED_NORM_MAX_ROWS = 16
SWAPPED_MIN_COLUMNS = 16384
#: Few-row products whose weight matrix has at least this many bytes go to the split-k tcgen05 kernel (the
#: second figure: with the LayerNorm fused in).  Measured on B200 inside whole decode steps, the split-k kernel
#: wins at every size of GPT-2's: its CTAs leave room on an SM for the next kernel's to begin ahead, and it
#: passes on the row statistics that the next LayerNorm needs.  The `mma.sync` kernel remains for the shapes
#: the split-k kernel refuses and for a LayerNorm of rows whose statistics nobody left.
SPLITK_MIN_WEIGHT_BYTES = 0
SPLITK_NORM_MIN_WEIGHT_BYTES = 0
_DEV_ERR = None


ROW_STATS_MAX_ROWS, ROW_STATS_MAX_WIDTH = 64, 8192


class RowStats:
    """Statistics of the float32 residual rows that a product has just written (per row and 32-column segment: sum
    and squared deviation from the segment's mean), kept so that the next product can apply a LayerNorm to those
    rows without reading them whole.  One buffer of fixed address (graphs capture it) on the device of the
    workspace that owns it; `of` says whose rows it describes: (the tensor, its torch version counter then, rows,
    width) or None.  The tensor is held, so its memory cannot be given to another tensor meanwhile.

    Who may trust them: a product of this module that is handed the same object and the same rows.  Who keeps them
    honest: every function of this module that writes a tensor and is handed the object forgets stale statistics;
    torch's in-place operations are seen by the version counter; and the block forgets them after any part that does
    not declare `leaves_row_stats` (parts/block.py), so a part that writes the residual with kernels of its own
    cannot leave them stale by omission."""

    def __init__(self, device):
        self.device = torch.device(device)
        self._buffer = None
        self.of = None

    def buffer(self) -> torch.Tensor:
        if self._buffer is None:
            self._buffer = torch.zeros(ROW_STATS_MAX_ROWS * (ROW_STATS_MAX_WIDTH // 32) * 2, dtype=torch.float32,
                                       device=self.device)
        return self._buffer

    def takes(self, rows: int, width: int) -> bool:
        return 0 < rows <= ROW_STATS_MAX_ROWS and width <= ROW_STATS_MAX_WIDTH

    def keep(self, t, rows: int, width: int) -> None:
        v = _version_of(t)
        self.of = (t, v, rows, width) if v >= 0 else None

    def forget(self) -> None:
        self.of = None

    def written(self, t) -> None:
        """`t` is being rewritten: statistics kept of it are stale."""
        if self.of is not None and t is not None and self.of[0].data_ptr() == t.data_ptr():
            self.of = None

    def describing(self, x, rows: int, width: int):
        """The statistics buffer if it describes exactly these rows as they are now, else None."""
        if self.of is None:
            return None
        held, version, n_rows, n_cols = self.of
        if held.data_ptr() == x.data_ptr() and _version_of(x) == version and (n_rows, n_cols) == (rows, width):
            return self._buffer
        return None


def _version_of(t) -> int:
    """torch's count of in-place changes of a tensor, or −1 where it is not kept (inference mode): then no
    statistics are kept either, since a change behind their back could not be seen."""
    try:
        return t._version
    except RuntimeError:
        return -1


def _splitk_takes(M: int, N: int, K: int, ldx: int, fused_norm: bool) -> bool:
    least = SPLITK_NORM_MIN_WEIGHT_BYTES if fused_norm else SPLITK_MIN_WEIGHT_BYTES
    if not USE_TCGEN05 or 2 * N * K < least or N >= SWAPPED_MIN_COLUMNS:
        return False
    from . import library
    return bool(library().vlrf_gemm_splitk_takes(M, N, K, ldx, 1 if fused_norm else 0))


def _dev_err() -> torch.Tensor:
    """The process-wide device error word for kernels whose callers pass none: int32 [1]; `device_errors()`
    reads and clears it."""
    global _DEV_ERR
    if _DEV_ERR is None:
        _DEV_ERR = torch.zeros(1, dtype=torch.int32, device="cuda")
    return _DEV_ERR


def set_chained_launch(on: bool) -> None:
    """Whether kernels are launched so that each may begin (fetch weights) while the one before it still
    runs.  On by default; off gives plain stream order."""
    call("vlrf_set_chained_launch", 1 if on else 0)


def device_errors() -> int:
    """Bits that kernels set in the shared error word since the last call (synchronises)."""
    if _DEV_ERR is None:
        return 0
    word = int(_DEV_ERR.item())
    if word:
        _DEV_ERR.zero_()
    return word


def sm_count() -> int:
    global _SM_COUNT
    if _SM_COUNT is None:
        import ctypes
        from . import library
        vals = [ctypes.c_int(0) for _ in range(4)]
        if library().vlrf_device_info(*[ctypes.byref(v) for v in vals]) != 0:
            raise KernelError("cannot query the device")
        _SM_COUNT = vals[0].value
    return _SM_COUNT


def _kv_args(kv_scatter, N: int) -> list:
    if kv_scatter is None:
        return [0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0]
    kc, vc, table, tok_slot, tok_pos, k_off, v_off, hkv, dh = kv_scatter
    _dev(kc, "k_cache", torch.bfloat16); _dev(vc, "v_cache", torch.bfloat16)
    _dev(table, "block_table", torch.int32); _dev(tok_slot, "tok_slot", torch.int32)
    _dev(tok_pos, "tok_pos", torch.int32)
    if kc.shape[1] != hkv or kc.shape[3] != dh or max(k_off, v_off) + hkv * dh > N:
        raise KernelError("cache scatter does not match the projection")
    return [_ptr(kc), _ptr(vc), _ptr(table), table.shape[1], _ptr(tok_slot), _ptr(tok_pos), k_off, v_off, hkv, dh,
            kc.shape[2]]


def _linear_dispatch(x, w, bias, out, act, residual, M, N, K, kv_scatter=None, stats=None) -> bool:
    bf16_out = out.dtype == torch.bfloat16
    if (x.dtype == torch.bfloat16 and M <= SKINNY_MAX_ROWS and K % 8 == 0 and USE_TCGEN05 and kv_scatter is None
            and N >= SWAPPED_MIN_COLUMNS):
        # few rows, very many columns (the head over the vocabulary): enough 128-row tiles of w to fill the GPU,
        # so w becomes the 128-row operand of the tcgen05 kernel and the rows of x its N
        call("vlrf_gemm_tcgen05", _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), M, N, K, K, N,
             dtype_code(out.dtype), act, *_kv_args(None, N), _ptr(_dev_err()), _stream())
        return False
    if x.dtype == torch.bfloat16 and M <= SKINNY_MAX_ROWS and _splitk_takes(M, N, K, K, False):
        # few rows, a large matrix: tiles of w on the tensor cores, the sum over k cut into parts
        scatter = kv_scatter is not None and bf16_out
        keep = stats is not None and not bf16_out and stats.takes(M, N)
        call("vlrf_gemm_splitk", _ptr(x), 0, _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), dtype_code(out.dtype),
             M, N, K, K, N, act, 0, 0, 0.0, *_kv_args(kv_scatter if scatter else None, N), 0,
             _ptr(stats.buffer()) if keep else 0, _ptr(_dev_err()), _stream())
        if keep:
            stats.keep(out, M, N)
        return scatter
    if x.dtype == torch.bfloat16 and M <= SKINNY_MAX_ROWS and K % 32 == 0:
        # few rows: the product is bound by streaming w once
        scatter = kv_scatter is not None and bf16_out
        call("vlrf_gemm_skinny", _ptr(x), 0, _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), dtype_code(out.dtype),
             M, N, K, K, N, act, 0, 0, 0.0, *_kv_args(kv_scatter if scatter else None, N), sm_count(), _ptr(_dev_err()),
             _stream())
        return scatter
    if x.dtype == torch.bfloat16 and K % 8 == 0 and USE_TCGEN05:
        # many rows: the tensor-core kernel (tcgen05, accumulator in tensor memory)
        scatter = kv_scatter is not None and bf16_out and kv_scatter[8] % 8 == 0 and kv_scatter[5] % 8 == 0
        call("vlrf_gemm_tcgen05", _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), M, N, K, K, N,
             dtype_code(out.dtype), act, *_kv_args(kv_scatter if scatter else None, N), _ptr(_dev_err()), _stream())
        return scatter
    call("vlrf_gemm_simt", _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), M, N, K, K, N,
         dtype_code(x.dtype), dtype_code(out.dtype), act, _stream())
    return False


def can_fuse_layernorm(n_rows: int, width: int, w_dtype: torch.dtype) -> bool:
    """Whether `linear_layernorm` takes this many rows of this width."""
    # with more rows, every CTA repeating the norm costs more than a norm kernel of its own
    if w_dtype != torch.bfloat16 or n_rows > FUSED_NORM_MAX_ROWS or n_rows < 1 or width % 32 != 0:
        return False
    from . import library
    return bool(library().vlrf_gemm_skinny_ln_fits(n_rows, width))


def linear_layernorm(x, gamma, beta, eps: float, w, bias, out, *, act=None, rows: int | None = None,
                     kv_scatter=None, stats: "RowStats | None" = None) -> None:
    """out = act(LayerNorm(x) · wᵀ + bias) for few rows, the norm fused into the product's prologue.
    x float32 [M,K]; w bfloat16 [N,K]; out bfloat16 or float32.  `kv_scatter` = (k_cache, v_cache,
    block_table, tok_slot, tok_pos, k_off, v_off, n_kv_heads, head_dim) also writes those columns of the
    result into one layer's paged cache."""
    _dev(x, "x", torch.float32); _dev(w, "w", torch.bfloat16); _dev(out, "out")
    _dev(gamma, "gamma", torch.float32); _dev(beta, "beta", torch.float32)
    M = x.shape[0] if rows is None else rows
    K, N = x.shape[1], w.shape[0]
    if w.shape[1] != K or out.shape[1] != N or out.shape[0] < M or gamma.shape[0] != K or beta.shape[0] != K:
        raise KernelError("linear_layernorm: sizes do not match")
    if bias is not None:
        _dev(bias, "bias", torch.float32)
    kv = _kv_args(kv_scatter, N)
    known = stats.describing(x, M, K) if stats is not None else None
    if stats is not None:
        stats.written(out)
    if known is not None and _splitk_takes(M, N, K, K, True):
        # the rows' statistics are at hand: each CTA normalises only the columns it multiplies
        call("vlrf_gemm_splitk", _ptr(x), 1, _ptr(w), _ptr(bias), 0, _ptr(out), dtype_code(out.dtype), M, N, K, K, N,
             ACT[act], _ptr(gamma), _ptr(beta), float(eps), *kv, _ptr(known), 0, _ptr(_dev_err()), _stream())
        return
    call("vlrf_gemm_skinny", _ptr(x), 1, _ptr(w), _ptr(bias), 0, _ptr(out), dtype_code(out.dtype), M, N, K, K, N,
         ACT[act], _ptr(gamma), _ptr(beta), float(eps), *kv, sm_count(), _ptr(_dev_err()), _stream())


def decode_splits(n_rows: int, n_heads: int, max_context: int) -> int:
    """Into how many parts a decode step cuts each context.  Measured inside whole steps of GPT-2 small,
    medium and XL: up to about 1.75 CTAs an SM in all, parts of at least 256 keys; more CTAs than that cost
    more (shared memory that the next kernel's CTAs would use, clusters to place) than they hide."""
    forced = os.environ.get("VLRF_B200_DECODE_SPLITS")
    if forced:
        return max(1, min(16, int(forced)))
    pairs = max(1, n_rows * n_heads)
    want = (7 * sm_count()) // (4 * pairs)
    return max(1, min(16, want, -(-max_context // 256)))


def attention_decode_needs_scratch(head_dim: int, n_split: int) -> bool:
    """Whether `attention_decode` with this split needs `partials` and `counters` (else the parts of a
    context merge inside a thread-block cluster)."""
    from . import library
    return bool(library().vlrf_attn_decode_needs_scratch(head_dim, n_split))


def attention_decode(qkv, q_off: int, k_cache, v_cache, block_table, tok_slot, tok_pos, out, n_rows: int,
                     n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int, n_split: int,
                     partials, counters, dev_err) -> None:
    """One query per row attends the keys 0…position of its slot; the context is cut into n_split parts.
    partials: float32 scratch of n_rows·n_heads·n_split·(head_dim+2); counters: int32 [n_rows·n_heads],
    zero between calls."""
    _dev(qkv, "qkv"); _dev(k_cache, "k_cache", qkv.dtype); _dev(v_cache, "v_cache", qkv.dtype)
    _dev(out, "out", qkv.dtype); _dev(block_table, "block_table", torch.int32)
    _dev(tok_slot, "tok_slot", torch.int32); _dev(tok_pos, "tok_pos", torch.int32)
    _dev(dev_err, "dev_err", torch.int32)
    nb, hkv, bt, dh = k_cache.shape
    if hkv != n_kv_heads or dh != head_dim or v_cache.shape != k_cache.shape:
        raise KernelError("attention_decode: cache shape does not match the heads")
    if out.shape[1] != n_heads * head_dim or out.shape[0] < n_rows or qkv.shape[0] < n_rows:
        raise KernelError("attention_decode: output does not match")
    if n_split > 1 and partials is not None:
        _dev(partials, "partials", torch.float32); _dev(counters, "counters", torch.int32)
        if partials.numel() < n_rows * n_heads * n_split * (head_dim + 2) or counters.numel() < n_rows * n_heads:
            raise KernelError("attention_decode: scratch is too small")
    call("vlrf_attn_decode", _ptr(qkv), dtype_code(qkv.dtype), qkv.shape[1], q_off, _ptr(k_cache), _ptr(v_cache), nb,
         _ptr(block_table), block_table.shape[1], _ptr(tok_slot), _ptr(tok_pos), _ptr(out), out.shape[1], n_rows,
         n_heads, n_kv_heads, head_dim, bt, float(scale), int(window), int(n_split), _ptr(partials), _ptr(counters),
         _ptr(dev_err), _stream())


def kv_append(qkv, k_off: int, v_off: int, k_cache, v_cache, block_table, tok_slot, tok_pos, n_tokens: int,
              n_kv_heads: int, head_dim: int, dev_err) -> None:
    """Scatter the K and V columns of qkv rows into one layer's paged cache
    [block, kv_head, block_tokens, head_dim]."""
    _dev(qkv, "qkv"); _dev(k_cache, "k_cache", qkv.dtype); _dev(v_cache, "v_cache", qkv.dtype)
    _dev(block_table, "block_table", torch.int32); _dev(tok_slot, "tok_slot", torch.int32)
    _dev(tok_pos, "tok_pos", torch.int32); _dev(dev_err, "dev_err", torch.int32)
    nb, hkv, bt, dh = k_cache.shape
    if hkv != n_kv_heads or dh != head_dim or v_cache.shape != k_cache.shape:
        raise KernelError("kv_append: cache shape does not match the heads")
    if qkv.shape[0] < n_tokens or tok_slot.shape[0] < n_tokens or tok_pos.shape[0] < n_tokens:
        raise KernelError("kv_append: fewer rows than tokens")
    ld = qkv.shape[1]
    if max(k_off, v_off) + n_kv_heads * head_dim > ld:
        raise KernelError("kv_append: K/V columns lie outside the row")
    call("vlrf_kv_append", _ptr(qkv), dtype_code(qkv.dtype), ld, k_off, v_off, _ptr(k_cache), _ptr(v_cache),
         _ptr(block_table), block_table.shape[1], _ptr(tok_slot), _ptr(tok_pos), n_tokens, n_kv_heads, head_dim,
         bt, _ptr(dev_err), _stream())


def attention_generic(qkv, q_off: int, k_cache, v_cache, block_table, tok_slot, tok_pos, out, n_tokens: int,
                      n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int, dev_err) -> None:
    """Each token's query attends the keys 0…position of its slot in the paged cache."""
    _dev(qkv, "qkv"); _dev(k_cache, "k_cache", qkv.dtype); _dev(v_cache, "v_cache", qkv.dtype)
    _dev(out, "out", qkv.dtype); _dev(block_table, "block_table", torch.int32)
    _dev(tok_slot, "tok_slot", torch.int32); _dev(tok_pos, "tok_pos", torch.int32)
    _dev(dev_err, "dev_err", torch.int32)
    nb, hkv, bt, dh = k_cache.shape
    if hkv != n_kv_heads or dh != head_dim or v_cache.shape != k_cache.shape:
        raise KernelError("attention: cache shape does not match the heads")
    if out.shape[1] != n_heads * head_dim or out.shape[0] < n_tokens or qkv.shape[0] < n_tokens:
        raise KernelError("attention: output does not match")
    if q_off + n_heads * head_dim > qkv.shape[1]:
        raise KernelError("attention: Q columns lie outside the row")
    call("vlrf_attn_generic", _ptr(qkv), dtype_code(qkv.dtype), qkv.shape[1], q_off, _ptr(k_cache), _ptr(v_cache),
         _ptr(block_table), block_table.shape[1], _ptr(tok_slot), _ptr(tok_pos), _ptr(out), out.shape[1],
         n_tokens, n_heads, n_kv_heads, head_dim, bt, float(scale), int(window), _ptr(dev_err), _stream())


def sample(logits, n_rows: int, out_tokens, *, temperature=None, top_k=None, top_p=None, rng_key=None,
           rng_ctr=None, next_tokens=None, next_pos=None, row_slot=None) -> None:
    """One token per row of float32 logits.  Rows with temperature ≤ 0 (or no temperature tensor at all)
    take the first maximal index; the others draw after top-k / top-p filtering.  `next_tokens`,
    `next_pos`, `row_slot` (int32 [n_rows], optional): the kernel also writes each token into next_tokens
    and adds one to next_pos where row_slot is not −1, which is all a decode session needs to go on."""
    _dev(logits, "logits", torch.float32); _dev(out_tokens, "out_tokens", torch.int32)
    V = logits.shape[1]
    if logits.shape[0] < n_rows or out_tokens.shape[0] < n_rows:
        raise KernelError("sample: fewer rows than asked for")
    if temperature is not None:
        _dev(temperature, "temperature", torch.float32)
        _dev(rng_key, "rng_key", torch.int64); _dev(rng_ctr, "rng_ctr", torch.int32)
    if top_k is not None:
        _dev(top_k, "top_k", torch.int32)
    if top_p is not None:
        _dev(top_p, "top_p", torch.float32)
    for name, t in (("next_tokens", next_tokens), ("next_pos", next_pos), ("row_slot", row_slot)):
        if t is not None:
            _dev(t, name, torch.int32)
            if t.shape[0] < n_rows:
                raise KernelError(f"sample: {name} has fewer rows than asked for")
    call("vlrf_sample", _ptr(logits), V, n_rows, V, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(rng_key),
         _ptr(rng_ctr), _ptr(out_tokens), _ptr(next_tokens), _ptr(next_pos), _ptr(row_slot), _stream())


def apply_penalties(logits, n_rows: int, generated, generated_len, *, repetition=None, frequency=None,
                    presence=None, no_repeat_ngram=None) -> None:
    """Edit logits in place from each row's generated tokens [n_rows, max_generated] and their count."""
    _dev(logits, "logits", torch.float32); _dev(generated, "generated", torch.int32)
    _dev(generated_len, "generated_len", torch.int32)
    for name, t, dt in (("repetition", repetition, torch.float32), ("frequency", frequency, torch.float32),
                        ("presence", presence, torch.float32), ("no_repeat_ngram", no_repeat_ngram, torch.int32)):
        if t is not None:
            _dev(t, name, dt)
    V = logits.shape[1]
    call("vlrf_apply_penalties", _ptr(logits), V, n_rows, V, _ptr(generated), generated.shape[1],
         _ptr(generated_len), _ptr(repetition), _ptr(frequency), _ptr(presence), _ptr(no_repeat_ngram), _stream())


def attention_prefill_takes(dtype: torch.dtype, head_dim: int, block_tokens: int, row_width: int, q_off: int) -> bool:
    """Whether the tensor-core prompt attention takes these sizes."""
    if dtype != torch.bfloat16:
        return False
    from . import library
    return bool(library().vlrf_attn_prefill_takes(head_dim, block_tokens, row_width, q_off))


def attention_prefill_kind(dtype: torch.dtype, head_dim: int, block_tokens: int, row_width: int, q_off: int, out_width: int) -> str:
    """Which kernel prompt attention of these sizes runs on: "tcgen05" (bfloat16, head size 64), "mma.sync"
    (bfloat16, head sizes 64 and 128) or "CUDA cores" (everything else, and the 32-bit path)."""
    from . import library
    lib = library()
    if dtype == torch.bfloat16 and PREFILL_ATTENTION_TCGEN05 and lib.vlrf_attn_prefill_tc_takes(head_dim, block_tokens, row_width, q_off, out_width):
        return "tcgen05"
    if dtype == torch.bfloat16 and lib.vlrf_attn_prefill_takes(head_dim, block_tokens, row_width, q_off):
        return "mma.sync"
    return "CUDA cores"


def attention_decode_kind(dtype: torch.dtype, head_dim: int) -> str:
    """Which kernel decode attention runs on: "mma.sync" (bfloat16, head size 64) or "CUDA cores"."""
    return "mma.sync" if dtype == torch.bfloat16 and head_dim == 64 else "CUDA cores"


def attention_prefill_parts(dtype: torch.dtype, n_seqs: int, max_new: int, n_heads: int, head_dim: int, block_tokens: int,
                            row_width: int, q_off: int) -> int:
    """Into how many parts `attention_prefill` best deals the keys of a long tile of queries (1: not at all;
    more want scratch, see there).  A tile's key blocks are a chain, so a step with few tiles is bound by its
    longest one (`tiles` blocks, for sequences that start at 0), not by the SMs: all blocks together, spread
    over the two CTAs that an SM holds, come to `even` blocks each, and parts pay when the chain is the longer
    of the two."""
    from . import library
    lib = library()
    if not PREFILL_ATTENTION_TCGEN05 or dtype != torch.bfloat16 \
            or not lib.vlrf_attn_prefill_tc_takes(head_dim, block_tokens, row_width, q_off, n_heads * head_dim):
        return 1
    tiles = -(-max_new // lib.vlrf_attn_prefill_tc_tile())
    even = tiles * (tiles + 1) / 2 * n_heads * n_seqs / (2 * sm_count())
    parts = int(tiles / (1.3 * max(even, lib.vlrf_attn_prefill_tc_min_part_blocks())) + 0.5)   # 1.3: a part's own cost
    if PREFILL_ATTENTION_PARTS is not None:
        parts = PREFILL_ATTENTION_PARTS
    return max(1, min(parts, lib.vlrf_attn_prefill_tc_max_parts()))


def attention_prefill_scratch(n_seqs: int, max_new: int, n_heads: int, n_parts: int) -> tuple[int, int]:
    """(float32 elements of `partials`, int32 elements of `counters`) that `attention_prefill` wants for
    n_parts > 1."""
    from . import library
    lib = library()
    tiles = -(-max_new // lib.vlrf_attn_prefill_tc_tile()) * n_seqs * n_heads
    return tiles * n_parts * lib.vlrf_attn_prefill_tc_part_floats(), tiles


def attention_prefill(qkv, q_off: int, k_cache, v_cache, block_table, seq_slot, seq_start, seq_pos0, out,
                      n_tokens: int, n_seqs: int, max_new: int, n_heads: int, n_kv_heads: int, head_dim: int,
                      scale: float, window: int, dev_err, n_parts: int = 1, partials=None, counters=None) -> None:
    """Causal attention of every sequence's new tokens (rows seq_start[i] … seq_start[i+1]−1 of qkv, the
    first of them at position seq_pos0[i]) over the sequence's cache, which already holds these tokens'
    keys and values.  bfloat16, head size 64 or 128.  n_parts > 1 (see attention_prefill_parts) deals the keys
    of long tiles to several CTAs and wants float32 `partials` and zeroed int32 `counters` of the sizes that
    attention_prefill_scratch gives; the counters are left zero."""
    _dev(qkv, "qkv", torch.bfloat16); _dev(k_cache, "k_cache", torch.bfloat16); _dev(v_cache, "v_cache", torch.bfloat16)
    _dev(out, "out", torch.bfloat16); _dev(block_table, "block_table", torch.int32)
    _dev(seq_slot, "seq_slot", torch.int32); _dev(seq_start, "seq_start", torch.int32)
    _dev(seq_pos0, "seq_pos0", torch.int32); _dev(dev_err, "dev_err", torch.int32)
    nb, hkv, bt, dh = k_cache.shape
    if hkv != n_kv_heads or dh != head_dim or v_cache.shape != k_cache.shape:
        raise KernelError("attention_prefill: cache shape does not match the heads")
    if out.shape[1] != n_heads * head_dim or out.shape[0] < n_tokens or qkv.shape[0] < n_tokens:
        raise KernelError("attention_prefill: output does not match")
    if seq_slot.shape[0] < n_seqs or seq_start.shape[0] < n_seqs + 1 or seq_pos0.shape[0] < n_seqs:
        raise KernelError("attention_prefill: sequence tables are too short")
    from . import library
    if PREFILL_ATTENTION_TCGEN05 and library().vlrf_attn_prefill_tc_takes(head_dim, bt, qkv.shape[1], q_off, out.shape[1]):
        # head size 64: S and O on the tcgen05 tensor cores, accumulators in tensor memory
        if n_parts > 1:
            _dev(partials, "partials", torch.float32); _dev(counters, "counters", torch.int32)
            want = attention_prefill_scratch(n_seqs, max_new, n_heads, n_parts)
            if partials.numel() < want[0] or counters.numel() < want[1]:
                raise KernelError("attention_prefill: scratch is too small for %d parts" % n_parts)
        call("vlrf_attn_prefill_tc", _ptr(qkv), qkv.shape[1], q_off, _ptr(k_cache), _ptr(v_cache), nb, _ptr(block_table),
             block_table.shape[1], _ptr(seq_slot), _ptr(seq_start), _ptr(seq_pos0), _ptr(out), out.shape[1], n_tokens,
             n_seqs, max_new, n_heads, n_kv_heads, head_dim, bt, float(scale), int(window), int(n_parts),
             _ptr(partials) if n_parts > 1 else 0, _ptr(counters) if n_parts > 1 else 0, _ptr(dev_err), _stream())
        return
    call("vlrf_attn_prefill", _ptr(qkv), qkv.shape[1], q_off, _ptr(k_cache), _ptr(v_cache), nb, _ptr(block_table),
         block_table.shape[1], _ptr(seq_slot), _ptr(seq_start), _ptr(seq_pos0), _ptr(out), out.shape[1], n_tokens, n_seqs,
         max_new, n_heads, n_kv_heads, head_dim, bt, float(scale), int(window), _ptr(dev_err), _stream())


# ---- RMS norm in groups, casts, gates ------------------------------------------------------------------------------

def group_rmsnorm(y, weight, eps: float, groups: int, out, rows=None, accumulate: bool = False, n_rows: int | None = None,
                  also=None) -> None:
    """out[r] (+)= y[rows[r] if rows is given else r] normed in `groups` equal consecutive parts (each divided by
    sqrt(mean(part²) + eps)) and multiplied by weight.  y float32; out float32 or bfloat16 (adding: float32 only).
    out may be y itself.  `also`: a bfloat16 tensor [rows, d] that receives the finished rows as well."""
    _rows(y, "y", torch.float32); _dev(weight, "weight", torch.float32); _dev(out, "out")
    d = y.shape[1]
    n = y.shape[0] if n_rows is None else n_rows
    if rows is not None:
        _dev(rows, "rows", torch.int32)
        n = rows.shape[0]
    if weight.shape[0] != d or out.shape[1] != d or out.shape[0] < n:
        raise KernelError("group_rmsnorm: sizes do not match")
    if also is not None:
        _dev(also, "also", torch.bfloat16)
        if also.shape[1] != d or also.shape[0] < n:
            raise KernelError("group_rmsnorm: the second output does not match")
    call("vlrf_group_rmsnorm", _ptr(y), y.stride(0), _ptr(rows), _ptr(weight), _ptr(out), dtype_code(out.dtype), d, n, d, int(groups),
         float(eps), 1 if accumulate else 0, _ptr(also), _stream())


def rmsnorm_shift(x, weight, mu, eps: float, state, ctx, out) -> None:
    """The plain RMS norm of the step's float32 residual rows followed by a token shift (see the kernel library's
    header): out[t] = n_t + (n_before − n_t) · mu.  state: float32 [slots, 2, d], the normed row of every sequence's last
    token, read and written by the parity of the positions."""
    _rows(x, "x", torch.float32); _dev(weight, "weight", torch.float32); _dev(mu, "mu", torch.float32)
    _dev(state, "state", torch.float32); _rows(out, "out")
    d, T = weight.shape[0], ctx.n_tokens
    if x.shape[1] < d or mu.shape[0] != d or out.shape[1] < d or min(x.shape[0], out.shape[0]) < T or state.dim() != 3 \
            or tuple(state.shape[1:]) != (2, d) or not state.is_contiguous():
        raise KernelError("rmsnorm_shift: sizes do not match")
    call("vlrf_rmsnorm_shift", _ptr(x), x.stride(0), _ptr(weight), _ptr(mu), float(eps), _ptr(state), _ptr(ctx.tok_slot),
         _ptr(ctx.tok_pos), _ptr(ctx.seq_start), ctx.n_seqs, T, _ptr(out), dtype_code(out.dtype), out.stride(0), d, _stream())


def add_row_vector(x, v, n_rows: int) -> None:
    """x[r] += v for the first n_rows float32 rows."""
    _rows(x, "x", torch.float32); _dev(v, "v", torch.float32)
    if x.shape[1] < v.shape[0] or x.shape[0] < n_rows:
        raise KernelError("add_row_vector: sizes do not match")
    call("vlrf_add_row_vector", _ptr(x), x.stride(0), _ptr(v), n_rows, v.shape[0], _stream())


def mingru_scan(proj, z_off: int, u_off: int, g_off: int, width: int, state, ctx, out) -> None:
    """The element-wise gated recurrence over the step's tokens (see the kernel library's header): proj float32 with the
    gate logits, candidate inputs and output gate logits at three column offsets; state float32 [slots, 2, width]."""
    _rows(proj, "proj", torch.float32); _dev(state, "state", torch.float32); _rows(out, "out")
    T = ctx.n_tokens
    if state.dim() != 3 or tuple(state.shape[1:]) != (2, width) or not state.is_contiguous() or out.shape[1] < width \
            or min(proj.shape[0], out.shape[0]) < T or proj.shape[1] < width + max(z_off, u_off, g_off):
        raise KernelError("mingru_scan: sizes do not match")
    call("vlrf_mingru_scan", _ptr(proj), proj.stride(0), z_off, u_off, g_off, width, _ptr(state), _ptr(ctx.seq_slot),
         _ptr(ctx.seq_start), _ptr(ctx.seq_pos0), ctx.n_seqs, ctx.max_new, _ptr(out), dtype_code(out.dtype), out.stride(0), _stream())


def cast_rows(x, out, n_rows: int) -> None:
    """The first n_rows float32 rows of x in out's dtype."""
    _dev(x, "x", torch.float32); _dev(out, "out")
    if out.shape[1] != x.shape[1] or min(out.shape[0], x.shape[0]) < n_rows:
        raise KernelError("cast_rows: sizes do not match")
    call("vlrf_cast_rows", _ptr(x), _ptr(out), dtype_code(out.dtype), n_rows * x.shape[1], _stream())


def gate_mul(a, b, out, gate: str, n_rows: int, cols: int, per: int = 1) -> None:
    """out[r, :cols] = gate(a[r, :cols]) · b[r, :cols]; gate "silu", "sigmoid" or "relu".  a, b and out may be column ranges
    of wider rows, and out may be a or b.  a and b may be float32 where out is bfloat16 (see the kernel library's header).
    per > 1: one column of a for every `per` consecutive columns of b (a gate per head on merged heads)."""
    for name, t in (("a", a), ("b", b), ("out", out)):
        _rows(t, name)
        if t.shape[0] < n_rows or t.shape[1] < (cols // per if name == "a" else cols):
            raise KernelError(f"gate_mul: {name} does not match")
    if per != 1:
        if per < 1 or cols % per != 0:
            raise KernelError(f"gate_mul: {cols} columns are no whole groups of {per}")
        call("vlrf_gate_mul_groups", _ptr(a), a.stride(0), dtype_code(a.dtype), _ptr(b), b.stride(0), dtype_code(b.dtype), _ptr(out),
             out.stride(0), dtype_code(out.dtype), n_rows, cols, int(per), GATE[gate], _stream())
        return
    call("vlrf_gate_mul", _ptr(a), a.stride(0), dtype_code(a.dtype), _ptr(b), b.stride(0), dtype_code(b.dtype), _ptr(out),
         out.stride(0), dtype_code(out.dtype), n_rows, cols, GATE[gate], _stream())


# ---- products per head and per group ---------------------------------------------------------------------------------
#: bfloat16 products per head and per group on the tcgen05 kernel where it takes the shape (off: the CUDA cores' kernels)
GROUPED_TCGEN05 = True


def linear_heads(x, w, out, n_rows: int) -> None:
    """out[m, h, :] = x[m, h, :] · w[h]ᵀ for every head.  x [M, H, K] and out [M, H, N] may be views into wider rows
    (strides (row, head, 1)); w [H, N, K] contiguous and of x's dtype; out float32 or x's dtype."""
    _dev(w, "w", x.dtype)
    H, N, K = w.shape
    for name, t, last in (("x", x, K), ("out", out, N)):
        if not t.is_cuda or t.dim() != 3 or t.stride(2) != 1 or t.shape[1] != H or t.shape[2] != last or t.shape[0] < n_rows:
            raise KernelError(f"linear_heads: {name} {list(t.shape)} does not match w {list(w.shape)}")
    if out.dtype not in (torch.float32, x.dtype):
        raise KernelError("linear_heads: the result is float32 or of the operands' dtype")
    if x.dtype == torch.bfloat16 and USE_TCGEN05 and GROUPED_TCGEN05 and x.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0:
        from . import library
        if library().vlrf_gemm_tcgen05_groups_takes(n_rows, H, N, K, x.stride(0), x.stride(1), out.stride(0), out.stride(1), 0):
            call("vlrf_gemm_tcgen05_groups", _ptr(x), x.stride(0), x.stride(1), _ptr(w), _ptr(out), out.stride(0), out.stride(1),
                 0, H, n_rows, N, K, dtype_code(out.dtype), 0, _ptr(_dev_err()), _stream())
            return
    call("vlrf_gemm_heads", _ptr(x), x.stride(0), x.stride(1), _ptr(w), _ptr(out), out.stride(0), out.stride(1), n_rows, N, K,
         H, dtype_code(x.dtype), dtype_code(out.dtype), _stream())


def linear_grouped(x, w, out, offsets, n_rows: int, act=None) -> None:
    """Rows offsets[g] … offsets[g+1]−1 of x [P, K] times w[g]ᵀ (w [G, N, K]) into the same rows of out [P, N];
    offsets: int32 [G + 1] on the device.  act: None, "gelu_tanh" or "relu2" on the result."""
    if act not in (None, "none", "gelu_tanh", "relu2"):
        raise KernelError(f"linear_grouped: activation '{act}' is not taken")
    _dev(x, "x"); _dev(w, "w", x.dtype); _dev(out, "out"); _dev(offsets, "offsets", torch.int32)
    G, N, K = w.shape
    if x.shape[1] != K or out.shape[1] != N or min(x.shape[0], out.shape[0]) < n_rows or offsets.numel() < G + 1:
        raise KernelError("linear_grouped: sizes do not match")
    if x.dtype == torch.bfloat16 and USE_TCGEN05 and GROUPED_TCGEN05 and n_rows > 0:
        from . import library
        if library().vlrf_gemm_tcgen05_groups_takes(n_rows, G, N, K, K, 0, N, 0, 1):
            call("vlrf_gemm_tcgen05_groups", _ptr(x), K, 0, _ptr(w), _ptr(out), N, 0, _ptr(offsets), G, n_rows, N, K,
                 dtype_code(out.dtype), ACT[act], _ptr(_dev_err()), _stream())
            return
    call("vlrf_gemm_grouped", _ptr(x), _ptr(w), _ptr(out), _ptr(offsets), G, n_rows, N, K, dtype_code(x.dtype),
         dtype_code(out.dtype), ACT[act], _stream())


# ---- attention over a cache of latents --------------------------------------------------------------------------------

def latent_append(proj, C: int, R: int, norm_weight, eps: float, inv_freq, rot_dims: int, cache, block_table, tok_slot,
                  tok_pos, n_tokens: int, dev_err, interleaved: bool = False) -> None:
    """Each token's row [RMSnorm(proj[:C]) · weight | rotate(proj[C:C+R])] into the paged cache [block, BT, row]."""
    _rows(proj, "proj", torch.float32); _dev(norm_weight, "norm_weight", torch.float32); _dev(cache, "cache")
    _dev(block_table, "block_table", torch.int32); _dev(tok_slot, "tok_slot", torch.int32)
    _dev(tok_pos, "tok_pos", torch.int32); _dev(dev_err, "dev_err", torch.int32)
    if inv_freq is not None:
        _dev(inv_freq, "inv_freq", torch.float32)
        if inv_freq.shape[0] < rot_dims // 2:
            raise KernelError("latent_append: the table of frequencies is too short")
    if proj.shape[1] < C + R or cache.shape[2] < C + R or norm_weight.shape[0] != C or proj.shape[0] < n_tokens:
        raise KernelError("latent_append: sizes do not match")
    call("vlrf_latent_append", _ptr(proj), proj.stride(0), C, R, _ptr(norm_weight), float(eps), _ptr(inv_freq), int(rot_dims),
         1 if interleaved else 0, _ptr(cache), dtype_code(cache.dtype), cache.shape[2], _ptr(block_table), block_table.shape[1], _ptr(tok_slot),
         _ptr(tok_pos), n_tokens, cache.shape[1], _ptr(dev_err), _stream())


def latent_q_rows(q, n_heads: int, dim: int, R: int, inv_freq, rot_dims: int, tok_pos, qn, qp, C: int, n_tokens: int,
                  interleaved: bool = False) -> None:
    """q float32 [T, H·(dim + R)] → qn [T, H·dim] (unrotated parts) and the last R columns of each head's C + R columns
    of qp (rotated parts, rotated by position)."""
    _rows(q, "q", torch.float32); _dev(qn, "qn"); _dev(qp, "qp", qn.dtype); _dev(tok_pos, "tok_pos", torch.int32)
    if inv_freq is not None:
        _dev(inv_freq, "inv_freq", torch.float32)
    if q.shape[1] != n_heads * (dim + R) or qn.shape[1] != n_heads * dim or qp.shape[1] != n_heads * (C + R):
        raise KernelError("latent_q_rows: sizes do not match")
    call("vlrf_latent_q_rows", _ptr(q), q.stride(0), n_heads, dim, R, _ptr(inv_freq), int(rot_dims), 1 if interleaved else 0, _ptr(tok_pos), _ptr(qn),
         qn.shape[1], _ptr(qp), qp.shape[1], C, dtype_code(qn.dtype), n_tokens, _stream())


#: the widest latent that the attention kernels over a latent cache hold
LATENT_MAX_RANK = 1024


def latent_gather(cache, C: int, R: int, block_table, tok_slot, tok_pos, out_c, out_r, n_tokens: int, dev_err) -> None:
    """The step's tokens' cache rows as plain matrices: latents out_c [T, C] and rotated key parts out_r [T, R]."""
    _dev(cache, "cache"); _dev(out_c, "out_c", cache.dtype); _dev(block_table, "block_table", torch.int32)
    _dev(tok_slot, "tok_slot", torch.int32); _dev(tok_pos, "tok_pos", torch.int32); _dev(dev_err, "dev_err", torch.int32)
    if R > 0:
        _dev(out_r, "out_r", cache.dtype)
    if cache.shape[2] < C + R or out_c.shape[1] != C or out_c.shape[0] < n_tokens or (R > 0 and (out_r.shape[1] != R or out_r.shape[0] < n_tokens)):
        raise KernelError("latent_gather: sizes do not match")
    call("vlrf_latent_gather", _ptr(cache), dtype_code(cache.dtype), cache.shape[2], C, R, _ptr(block_table), block_table.shape[1],
         _ptr(tok_slot), _ptr(tok_pos), _ptr(out_c), _ptr(out_r) if R > 0 else 0, n_tokens, cache.shape[1], _ptr(dev_err), _stream())


#: prompt steps whose sequences all begin at position 0 form keys and values and run the kernel over plain rows (off: the
#: latent-space kernels take every step)
LATENT_PROMPT_ROWS = True


def attention_rows_takes(dtype: torch.dtype, dim: int, R: int, vdim: int, n_heads: int) -> bool:
    if dtype != torch.bfloat16 or not LATENT_PROMPT_ROWS:
        return False
    from . import library
    # (as the mixer lays them out: keys and values are column ranges of one product's rows)
    return (n_heads * dim) % 8 == 0 and bool(library().vlrf_attn_rows_takes(
        dim, R, vdim, n_heads * dim, n_heads * R, n_heads * (dim + vdim), R, n_heads * (dim + vdim), n_heads * vdim))


def attention_rows_strides_ok(dim: int, R: int, vdim: int, ld_qn: int, ld_qr: int, ld_kn: int, ld_kr: int, ld_v: int, ld_out: int) -> bool:
    from . import library
    return bool(library().vlrf_attn_rows_takes(dim, R, vdim, ld_qn, ld_qr, ld_kn, ld_kr, ld_v, ld_out))


def attention_rows(qn, qr, kn, kr, v, seq_start, out, n_seqs: int, max_new: int, n_heads: int, dim: int, R: int, vdim: int,
                   scale: float) -> None:
    """Causal attention of sequences that begin at position 0 over keys and values in plain rows (see the kernel library's
    header): qn, kn [T, H·dim]; qr [T, H·R], kr [T, R] (None with R = 0); v, out [T, H·vdim]; bfloat16."""
    for name, t in (("qn", qn), ("kn", kn), ("v", v), ("out", out)):          # (column ranges of wider rows are taken)
        _rows(t, name, torch.bfloat16)
    if R > 0:
        _rows(qr, "qr", torch.bfloat16); _rows(kr, "kr", torch.bfloat16)
    _dev(seq_start, "seq_start", torch.int32)
    if qn.shape[1] != n_heads * dim or kn.shape[1] != n_heads * dim or v.shape[1] != n_heads * vdim or out.shape[1] != n_heads * vdim \
            or (R > 0 and (qr.shape[1] != n_heads * R or kr.shape[1] != R)) or seq_start.shape[0] < n_seqs + 1:
        raise KernelError("attention_rows: sizes do not match")
    lib_takes = attention_rows_strides_ok(dim, R, vdim, qn.stride(0), qr.stride(0) if R > 0 else 8, kn.stride(0), kr.stride(0) if R > 0 else 8,
                                          v.stride(0), out.stride(0))
    if not lib_takes:
        raise KernelError("attention_rows: these sizes or row strides are not taken")
    call("vlrf_attn_rows", _ptr(qn), qn.stride(0), _ptr(qr) if R > 0 else 0, qr.stride(0) if R > 0 else 0, _ptr(kn), kn.stride(0),
         _ptr(kr) if R > 0 else 0, kr.stride(0) if R > 0 else 0, _ptr(v), v.stride(0), _ptr(seq_start), _ptr(out), out.stride(0), n_seqs, max_new, n_heads, dim, R, vdim, float(scale), _stream())


LATENT_ATTENTION_MMA = True          # off: every step takes the general kernel (for measurements and cross-checks)


def _latent_mma_takes(dtype: torch.dtype, C: int, R: int, row_w: int, block_tokens: int, ld_q: int) -> bool:
    if dtype != torch.bfloat16 or not LATENT_ATTENTION_MMA:
        return False
    from . import library
    return bool(library().vlrf_attn_latent_mma_takes(C, R, row_w, block_tokens, ld_q))


def attention_latent_kind(dtype: torch.dtype, C: int, R: int) -> dict:
    """Which kernels attention over a latent cache of these sizes runs on: "mma.sync" or "CUDA cores"."""
    kind = "mma.sync" if _latent_mma_takes(dtype, C, R, C + R, 64, 8) else "CUDA cores"
    return {"prompt": kind, "decode": kind}


def latent_decode_splits(n_rows: int, n_heads: int, max_context: int, C: int, R: int) -> int:
    """Into how many parts a decode step cuts each context over a latent cache: as many as keep all CTAs on the SMs at
    one time (a part more, and the step runs a second, nearly empty wave: 64 rows × 5 parts on 296 places took 50 µs,
    × 4 parts 45 µs), at most 8, parts of at least 64 rows."""
    forced = os.environ.get("VLRF_B200_DECODE_SPLITS")
    if forced:
        return max(1, min(16, int(forced)))
    from . import library
    ctas = max(1, n_rows * ((n_heads + 15) // 16))
    places = sm_count() * library().vlrf_attn_latent_mma_ctas_per_sm(C, R)
    return max(1, min(8, places // ctas, -(-max_context // 64)))


def attention_latent(qp, cache, C: int, R: int, block_table, tok_slot, tok_pos, out, n_tokens: int, n_heads: int, scale: float,
                     window: int, dev_err, ctx=None) -> None:
    """Each token's heads (queries in latent space, [T, H·(C + R)]) attend the rows 0…position of the token's slot in
    the latent cache [block, BT, row]; out [T, H·C] receives Σ_j p_j c_j per head.  With the step's context (`ctx`:
    its sequence tables and scratch) bfloat16 steps of sizes that the tensor-core kernel takes run there."""
    _dev(qp, "qp"); _dev(cache, "cache", qp.dtype); _dev(out, "out", qp.dtype)
    _dev(block_table, "block_table", torch.int32); _dev(tok_slot, "tok_slot", torch.int32)
    _dev(tok_pos, "tok_pos", torch.int32); _dev(dev_err, "dev_err", torch.int32)
    if qp.shape[1] != n_heads * (C + R) or out.shape[1] != n_heads * C or cache.shape[2] < C + R \
            or min(qp.shape[0], out.shape[0]) < n_tokens:
        raise KernelError("attention_latent: sizes do not match")
    if ctx is not None and _latent_mma_takes(qp.dtype, C, R, cache.shape[2], cache.shape[1], qp.shape[1]):
        n_split, partials = 1, None
        if ctx.max_new == 1:
            n_split = latent_decode_splits(ctx.n_seqs, n_heads, ctx.max_context, C, R)
            if n_split > 1:
                partials = ctx.ws.get("latent_attn_partials", ctx.n_seqs * ((n_heads + 15) // 16) * n_split * 16, C + 2, torch.float32)
        call("vlrf_attn_latent_mma", _ptr(qp), qp.shape[1], _ptr(cache), cache.shape[2], C, R, _ptr(block_table),
             block_table.shape[1], _ptr(ctx.seq_slot), _ptr(ctx.seq_start), _ptr(ctx.seq_pos0), _ptr(out), out.shape[1],
             ctx.n_seqs, ctx.max_new, n_heads, cache.shape[1], float(scale), int(window), n_split, _ptr(partials),
             _ptr(dev_err), _stream())
        return
    call("vlrf_attn_latent", _ptr(qp), dtype_code(qp.dtype), qp.shape[1], _ptr(cache), cache.shape[2], C, R, _ptr(block_table),
         block_table.shape[1], _ptr(tok_slot), _ptr(tok_pos), _ptr(out), out.shape[1], n_tokens, n_heads, cache.shape[1],
         float(scale), int(window), _ptr(dev_err), _stream())


# ---- routed experts --------------------------------------------------------------------------------------------------

#: the most router outputs that the routing kernels take
MOE_MAX_OUTPUTS = 512


def moe_route(z, n_experts: int, top: int, shared_gate: bool, tok_slot, ids, wts, rank, gate, counts, n_tokens: int) -> None:
    """From float32 router logits z [T, ≥ E (+1)]: ids, wts, rank [T, top], gate [T] (see the kernel library's header)."""
    _rows(z, "z", torch.float32); _dev(ids, "ids", torch.int32); _dev(wts, "wts", torch.float32)
    _dev(rank, "rank", torch.int32); _dev(counts, "counts", torch.int32)
    if gate is not None:
        _dev(gate, "gate", torch.float32)
    if tok_slot is not None:
        _dev(tok_slot, "tok_slot", torch.int32)
    if z.shape[0] < n_tokens or ids.numel() < n_tokens * top or counts.numel() < n_experts:
        raise KernelError("moe_route: sizes do not match")
    if z.shape[1] < n_experts + (1 if shared_gate else 0):
        raise KernelError("moe_route: the logits' rows are too short")
    call("vlrf_moe_route", _ptr(z), z.stride(0), n_experts, top, 1 if shared_gate else 0, _ptr(tok_slot), _ptr(ids), _ptr(wts),
         _ptr(rank), _ptr(gate), _ptr(counts), n_tokens, _stream())


def moe_route_scored(z, n_outputs: int, top: int, groups: int, keep: int, n_identity: int, scale: float, correction, tok_slot,
                     ids, wts, rank, counts, n_tokens: int, scoring: str = "softmax") -> None:
    """From float32 router logits z [T, ≥ n_outputs]: softmax over all outputs (scoring "sigmoid": the sigmoid of each),
    the choice by score + correction inside the `keep` best of `groups` groups, weights score · scale; the last
    n_identity outputs get id −2 and no rank (see the kernel library's header)."""
    if scoring not in ("softmax", "sigmoid"):
        raise KernelError(f"moe_route_scored: scoring '{scoring}' is neither 'softmax' nor 'sigmoid'")
    _rows(z, "z", torch.float32); _dev(ids, "ids", torch.int32); _dev(wts, "wts", torch.float32)
    _dev(rank, "rank", torch.int32); _dev(counts, "counts", torch.int32); _dev(correction, "correction", torch.float32)
    if tok_slot is not None:
        _dev(tok_slot, "tok_slot", torch.int32)
    if z.shape[0] < n_tokens or z.shape[1] < n_outputs or ids.numel() < n_tokens * top or correction.numel() < n_outputs \
            or counts.numel() < max(n_outputs - n_identity, 1):
        raise KernelError("moe_route_scored: sizes do not match")
    call("vlrf_moe_route_scored", _ptr(z), z.stride(0), n_outputs, top, int(groups), int(keep), int(n_identity), float(scale),
         1 if scoring == "sigmoid" else 0, _ptr(correction), _ptr(tok_slot), _ptr(ids), _ptr(wts), _ptr(rank), _ptr(counts), n_tokens, _stream())


def moe_plan(counts, offsets, n_experts: int) -> None:
    _dev(counts, "counts", torch.int32); _dev(offsets, "offsets", torch.int32)
    if counts.numel() < n_experts or offsets.numel() < n_experts + 1:
        raise KernelError("moe_plan: sizes do not match")
    call("vlrf_moe_plan", _ptr(counts), _ptr(offsets), n_experts, _stream())


def moe_gather(h, ids, rank, offsets, sorted_rows, row_of, n_tokens: int, top: int) -> None:
    _dev(h, "h"); _dev(sorted_rows, "sorted_rows", h.dtype); _dev(row_of, "row_of", torch.int32)
    if sorted_rows.shape[1] != h.shape[1] or sorted_rows.shape[0] < n_tokens * top or h.shape[0] < n_tokens:
        raise KernelError("moe_gather: sizes do not match")
    call("vlrf_moe_gather", _ptr(h), dtype_code(h.dtype), h.shape[1], _ptr(ids), _ptr(rank), _ptr(offsets), _ptr(sorted_rows),
         _ptr(row_of), n_tokens, top, _stream())


def moe_combine(expert_out, row_of, wts, top: int, shared_out, gate, y, n_tokens: int, residual=None, ids=None, h=None) -> None:
    """y[t] = Σ_j wts[t, j] · expert_out[row_of[t, j]] (+ gate[t] · shared_out[t]) (+ residual[t]), float32.  With `ids` and
    the experts' input rows `h`: a pair whose id is −2 (an expert that returns its input) adds wts[t, j] · h[t]."""
    _dev(expert_out, "expert_out", torch.float32); _dev(y, "y", torch.float32)
    if (ids is None) != (h is None):
        raise KernelError("moe_combine: experts that return their input need ids and the input rows")
    if h is not None:
        _dev(ids, "ids", torch.int32); _dev(h, "h")
        if h.shape[1] != y.shape[1] or h.shape[0] < n_tokens or not h.is_contiguous():
            raise KernelError("moe_combine: the input rows do not match")
    if shared_out is not None:
        _dev(shared_out, "shared_out", torch.float32)
    if y.shape[1] != expert_out.shape[1] or y.shape[0] < n_tokens:
        raise KernelError("moe_combine: sizes do not match")
    call("vlrf_moe_combine", _ptr(expert_out), expert_out.shape[1], _ptr(row_of), _ptr(wts), top, _ptr(shared_out), _ptr(gate),
         _ptr(residual), _ptr(y), n_tokens, _ptr(ids), _ptr(h), dtype_code(h.dtype) if h is not None else 0, _stream())


# ---- a residual in several streams -------------------------------------------------------------------------------------

def embed_streams(table, tokens, out, streams: int, scale: float, dev_err) -> None:
    """out[t, s·d …] = table[tokens[t]] · scale for every stream s: float32 [T, streams·d]."""
    _dev(table, "table"); _dev(tokens, "tokens", torch.int32); _dev(out, "out", torch.float32)
    _dev(dev_err, "dev_err", torch.int32)
    T = tokens.shape[0]
    V, d = table.shape
    if out.shape[0] < T or out.shape[1] != streams * d:
        raise KernelError("embed_streams: output does not match")
    call("vlrf_embed_streams", _ptr(table), dtype_code(table.dtype), _ptr(tokens), _ptr(out), T, d, V, int(streams), float(scale),
         _ptr(dev_err), _stream())


def streams_read_norm(x, streams: int, coefficients, weight, eps: float, out, rows=None, n_rows: int | None = None) -> None:
    """out[r] = RMSnorm(Σ_s coefficients[s] · x[row, s]) · weight, row = rows[r] if rows is given else r; coefficients
    None: the plain sum.  x float32 [·, streams·d]; out float32 or bfloat16 [n, d]."""
    _dev(x, "x", torch.float32); _dev(weight, "weight", torch.float32); _dev(out, "out")
    d = weight.shape[0]
    n = x.shape[0] if n_rows is None else n_rows
    if rows is not None:
        _dev(rows, "rows", torch.int32)
        n = rows.shape[0]
    if coefficients is not None:
        _dev(coefficients, "coefficients", torch.float32)
        if coefficients.numel() != streams:
            raise KernelError("streams_read_norm: one coefficient per stream")
    if x.shape[1] != streams * d or out.shape[1] != d or out.shape[0] < n:
        raise KernelError("streams_read_norm: sizes do not match")
    call("vlrf_streams_read_norm", _ptr(x), _ptr(rows), _ptr(coefficients), _ptr(weight), _ptr(out), dtype_code(out.dtype), n, d,
         int(streams), float(eps), _stream())


def streams_write(x, streams: int, mix, out_coefficients, y, n_rows: int) -> None:
    """x[t, j] ← Σ_s mix[s, j] · x[t, s] + out_coefficients[j] · y[t], every stream j at once from the old ones."""
    _dev(x, "x", torch.float32); _dev(y, "y", torch.float32); _dev(mix, "mix", torch.float32)
    _dev(out_coefficients, "out_coefficients", torch.float32)
    d = y.shape[1]
    if x.shape[1] != streams * d or tuple(mix.shape) != (streams, streams) or out_coefficients.numel() != streams \
            or min(x.shape[0], y.shape[0]) < n_rows:
        raise KernelError("streams_write: sizes do not match")
    call("vlrf_streams_write", _ptr(x), _ptr(mix), _ptr(out_coefficients), _ptr(y), n_rows, d, int(streams), _stream())


def streams_write_read(x, streams: int, mix, out_coefficients, y, coefficients, weight, eps: float, out, n_rows: int) -> None:
    """`streams_write` followed by `streams_read_norm` of the same rows with the next sublayer's coefficients and norm
    weight, in one pass over the streams."""
    _dev(x, "x", torch.float32); _dev(y, "y", torch.float32); _dev(mix, "mix", torch.float32); _dev(out, "out")
    _dev(out_coefficients, "out_coefficients", torch.float32); _dev(coefficients, "coefficients", torch.float32)
    _dev(weight, "weight", torch.float32)
    d = y.shape[1]
    if x.shape[1] != streams * d or tuple(mix.shape) != (streams, streams) or out_coefficients.numel() != streams \
            or coefficients.numel() != streams or weight.shape[0] != d or out.shape[1] != d or min(x.shape[0], y.shape[0], out.shape[0]) < n_rows:
        raise KernelError("streams_write_read: sizes do not match")
    call("vlrf_streams_write_read", _ptr(x), _ptr(mix), _ptr(out_coefficients), _ptr(y), _ptr(coefficients), _ptr(weight), _ptr(out),
         dtype_code(out.dtype), n_rows, d, int(streams), float(eps), _stream())


def softcap(values, n_rows: int, cap: float) -> None:
    """values[:n_rows] ← cap · tanh(values / cap), float32, in place."""
    _dev(values, "values", torch.float32)
    call("vlrf_softcap", _ptr(values), n_rows * values.shape[1], float(cap), _stream())


def embed_bigram(table, pairs, buckets: int, mul_prev: int, mul_cur: int, scale: float, kept, ctx, out, also=None) -> None:
    """out[t] = table[token] · scale + pairs[(token before · mul_prev + token · mul_cur) mod buckets] (pairs[buckets] for a
    sequence's first token): float32 [T, d].  kept: int32 [slots, 2], every sequence's last token by the parity of its
    length (see the kernel library's header).  also: a bfloat16 tensor [T, d] that receives the rows' rounding as well."""
    _dev(table, "table"); _dev(pairs, "pairs", table.dtype); _dev(kept, "kept", torch.int32); _dev(out, "out", torch.float32)
    if also is not None:
        _dev(also, "also", torch.bfloat16)
        if also.shape[0] < ctx.n_tokens or also.shape[1] != table.shape[1]:
            raise KernelError("embed_bigram: the second output does not match")
    V, d = table.shape
    if tuple(pairs.shape) != (buckets + 1, d) or out.shape[0] < ctx.n_tokens or out.shape[1] != d or kept.dim() != 2 \
            or kept.shape[1] != 2 or not kept.is_contiguous():
        raise KernelError("embed_bigram: sizes do not match")
    call("vlrf_embed_bigram", _ptr(table), _ptr(pairs), dtype_code(table.dtype), _ptr(ctx.tokens), _ptr(ctx.tok_slot), _ptr(ctx.tok_pos),
         _ptr(ctx.seq_start), ctx.n_seqs, _ptr(kept), _ptr(out), ctx.n_tokens, d, V, int(buckets), int(mul_prev), int(mul_cur),
         float(scale), _ptr(also), _ptr(ctx.dev_err), _stream())


def scale_values(values, n_rows: int, factor: float) -> None:
    """values[:n_rows] ← values · factor, float32, in place."""
    _dev(values, "values", torch.float32)
    call("vlrf_scale_values", _ptr(values), n_rows * values.shape[1], float(factor), _stream())


def gate_mul_clamped(a, b, out, limit: float, alpha: float, n_rows: int, cols: int) -> None:
    """out[r, :cols] = g · sigmoid(alpha · g) · (u + 1) with g = min(a, limit), u = clamp(b, −limit, limit); a, b and out may be
    column ranges of wider rows, and out may be a or b."""
    for name, t in (("a", a), ("b", b), ("out", out)):
        _rows(t, name)
        if t.shape[0] < n_rows or t.shape[1] < cols:
            raise KernelError(f"gate_mul_clamped: {name} does not match")
    call("vlrf_gate_mul_clamped", _ptr(a), a.stride(0), dtype_code(a.dtype), _ptr(b), b.stride(0), dtype_code(b.dtype), _ptr(out),
         out.stride(0), dtype_code(out.dtype), n_rows, cols, float(limit), float(alpha), _stream())


# ---- attention with key and value sizes of their own ---------------------------------------------------------------------

def qkv_rope_append(proj, q_off: int, k_off: int, v_off: int, freq, rot: int, q_out, k_cache, v_cache, block_table, tok_slot,
                    tok_pos, n_tokens: int, n_heads: int, n_kv_heads: int, dk: int, dv: int, write_cache: bool, dev_err, *,
                    norm: str | None = None, q_norm=None, k_norm=None, eps: float = 0.0, interleaved: bool = False,
                    magnitude: float = 1.0) -> None:
    """Queries (rotated) into q_out, keys (rotated) and values into the paged cache, from the float32 rows of a layer's
    input product.  proj may be a range of columns of wider rows.  norm "head" / "all": an RMS norm of queries and keys
    ahead of the rotation, every head by itself (weights of dk entries shared by the heads) or the whole projection as
    one row (weights of heads · dk entries); interleaved: entry 2i pairs with 2i + 1; magnitude: a factor on cosines and
    sines.  With write_cache False the key and value columns are not read (k_off, v_off, k_norm are ignored)."""
    _rows(proj, "proj", torch.float32); _dev(q_out, "q_out"); _dev(k_cache, "k_cache", q_out.dtype); _dev(v_cache, "v_cache", q_out.dtype)
    _dev(block_table, "block_table", torch.int32); _dev(tok_slot, "tok_slot", torch.int32); _dev(tok_pos, "tok_pos", torch.int32)
    nb, hkv, bt, kd = k_cache.shape
    if hkv != n_kv_heads or kd != dk or tuple(v_cache.shape) != (nb, hkv, bt, dv):
        raise KernelError("qkv_rope_append: cache shape does not match the heads")
    if rot > 0:
        _dev(freq, "freq", torch.float32)
        if freq.numel() != rot // 2:
            raise KernelError("qkv_rope_append: one frequency per rotated pair")
    if proj.shape[0] < n_tokens or q_out.shape[0] < n_tokens:
        raise KernelError("qkv_rope_append: fewer rows than tokens")
    code = {None: 0, "head": 1, "all": 2}.get(norm, -1)
    if code < 0:
        raise KernelError(f"qkv_rope_append: norm '{norm}' is neither 'head' nor 'all'")
    if code:
        _dev(q_norm, "q_norm", torch.float32)
        if q_norm.numel() != (dk if code == 1 else n_heads * dk):
            raise KernelError("qkv_rope_append: the queries' norm weights do not match")
        if write_cache:
            _dev(k_norm, "k_norm", torch.float32)
            if k_norm.numel() != (dk if code == 1 else n_kv_heads * dk):
                raise KernelError("qkv_rope_append: the keys' norm weights do not match")
    call("vlrf_qkv_norm_rope_append", _ptr(proj), proj.stride(0), q_off, k_off if write_cache else 0, v_off if write_cache else 0,
         _ptr(freq) if rot > 0 else 0, int(rot), _ptr(q_out), q_out.shape[1], _ptr(k_cache), _ptr(v_cache), dtype_code(q_out.dtype),
         _ptr(block_table), block_table.shape[1], _ptr(tok_slot), _ptr(tok_pos), n_tokens, n_heads, n_kv_heads, dk, dv, bt,
         1 if write_cache else 0, code, _ptr(q_norm) if code else 0, _ptr(k_norm) if code and write_cache else 0, float(eps),
         1 if interleaved else 0, float(magnitude), _ptr(dev_err), _stream())


def _check_head_gate(gate, n_rows: int, n_heads: int) -> None:
    if gate is not None:
        _rows(gate, "gate", torch.float32)
        if gate.shape[0] < n_rows or gate.shape[1] < n_heads:
            raise KernelError("attention_window: the gate has one float32 logit per token and query head")


def attention_window(q, k_cache, v_cache, block_table, tok_slot, tok_pos, out, n_tokens: int, n_heads: int, n_kv_heads: int,
                     dk: int, dv: int, scale: float, window: int, out_scale: float, dev_err, *, softcap: float = 0.0,
                     keep_first: int = 0, sink=None, gate=None) -> None:
    """Each token's queries attend the visible keys of its slot; out may be a range of columns of wider rows.  softcap > 0
    squashes the scaled scores; keys at positions below keep_first stay visible whatever the window; sink: float32
    [heads], exp(sink) joins the softmax's denominator; gate: float32 [T, ≥ heads] (a range of columns of wider rows will
    do), head h's result times sigmoid(gate[t, h])."""
    _check_head_gate(gate, n_tokens, n_heads)
    if sink is not None:
        _dev(sink, "sink", torch.float32)
        if sink.numel() != n_heads:
            raise KernelError("attention_window: one sink per query head")
    _dev(q, "q"); _dev(k_cache, "k_cache", q.dtype); _dev(v_cache, "v_cache", q.dtype); _rows(out, "out", q.dtype)
    _dev(block_table, "block_table", torch.int32); _dev(tok_slot, "tok_slot", torch.int32); _dev(tok_pos, "tok_pos", torch.int32)
    nb, hkv, bt, kd = k_cache.shape
    if hkv != n_kv_heads or kd != dk or tuple(v_cache.shape) != (nb, hkv, bt, dv):
        raise KernelError("attention_window: cache shape does not match the heads")
    if out.shape[1] < n_heads * dv or out.shape[0] < n_tokens or q.shape[0] < n_tokens:
        raise KernelError("attention_window: output does not match")
    call("vlrf_attn_window_ex", _ptr(q), dtype_code(q.dtype), q.shape[1], _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
         block_table.shape[1], _ptr(tok_slot), _ptr(tok_pos), _ptr(out), out.stride(0), n_tokens, n_heads, n_kv_heads, dk, dv, bt,
         float(scale), int(window), float(out_scale), float(softcap), int(keep_first), _ptr(sink), _ptr(gate),
         gate.stride(0) if gate is not None else 0, _ptr(dev_err), _stream())


# ---- a state-space recurrence with a matrix state per head -----------------------------------------------------------------

def ssd_conv(proj, x_off: int, weight, bias, state, conv_off: int, seq_slot, seq_start, seq_pos0, out, n_seqs: int, max_new: int) -> None:
    """Causal convolution with bias and x·sigmoid(x) over `channels` columns of proj from x_off; leaves the last taps − 1
    inputs of every sequence in its state row.  state float32 [slots, 2, state_row]."""
    _rows(proj, "proj", torch.float32); _dev(weight, "weight", torch.float32); _dev(bias, "bias", torch.float32)
    _dev(state, "state", torch.float32); _dev(out, "out", torch.float32)
    channels, taps = weight.shape
    if out.shape[1] != channels or bias.shape[0] != channels or state.dim() != 3 or state.shape[1] != 2:
        raise KernelError("ssd_conv: sizes do not match")
    call("vlrf_ssd_conv", _ptr(proj), proj.stride(0), x_off, _ptr(weight), _ptr(bias), _ptr(state), state.shape[2], conv_off,
         _ptr(seq_slot), _ptr(seq_start), _ptr(seq_pos0), _ptr(out), n_seqs, max_new, channels, taps, _stream())


def ssd_scan(xbc, proj, dt_off: int, dt_bias, a_log, d_skip, state, seq_slot, seq_start, seq_pos0, y, n_seqs: int, n_heads: int,
             n_groups: int, n_state: int, p: int, max_new: int = 16) -> None:
    """The recurrence over every sequence's new tokens, from and into the state rows; y float32 [T, heads·p]."""
    _dev(xbc, "xbc", torch.float32); _rows(proj, "proj", torch.float32); _dev(state, "state", torch.float32); _dev(y, "y", torch.float32)
    for name, t in (("dt_bias", dt_bias), ("a_log", a_log), ("d_skip", d_skip)):
        _dev(t, name, torch.float32)
        if t.numel() != n_heads:
            raise KernelError(f"ssd_scan: {name} has one number per head")
    if y.shape[1] != n_heads * p or state.dim() != 3 or state.shape[1] != 2:
        raise KernelError("ssd_scan: sizes do not match")
    call("vlrf_ssd_scan", _ptr(xbc), xbc.shape[1], _ptr(proj), proj.stride(0), dt_off, _ptr(dt_bias), _ptr(a_log), _ptr(d_skip),
         _ptr(state), state.shape[2], _ptr(seq_slot), _ptr(seq_start), _ptr(seq_pos0), _ptr(y), n_seqs, int(max_new), n_heads, n_groups,
         n_state, p, _stream())


def ssd_gate_norm(y, proj, z_off: int, weight, groups: int, eps: float, factor: float, out, n_rows: int) -> None:
    """out[r] = factor · groupnorm(y[r] · silu(proj[r, z_off …])) · weight; out may be a range of columns of wider rows."""
    _dev(y, "y", torch.float32); _rows(proj, "proj", torch.float32); _dev(weight, "weight", torch.float32); _rows(out, "out")
    d = y.shape[1]
    if weight.shape[0] != d or out.shape[1] < d or min(y.shape[0], proj.shape[0], out.shape[0]) < n_rows:
        raise KernelError("ssd_gate_norm: sizes do not match")
    call("vlrf_ssd_gate_norm", _ptr(y), _ptr(proj), proj.stride(0), z_off, _ptr(weight), _ptr(out), dtype_code(out.dtype), out.stride(0),
         n_rows, d, int(groups), float(eps), float(factor), _stream())


#: largest head size of the attention with key and value sizes of their own; most taps and largest value size of the
#: state-space kernels
WINDOW_HEAD_MAX, SSD_MAX_TAPS, SSD_MAX_VDIM, SSD_MAX_STATE = 256, 16, 4096, 512


#: bfloat16 attention with key and value sizes of their own on the tensor cores where the kernel takes the sizes (off: the
#: CUDA cores' kernel, which takes everything)
WINDOW_ATTENTION_MMA = True


def _window_mma_takes(dtype, n_heads: int, n_kv_heads: int, dk: int, dv: int, bt: int, ldq: int, ld_out: int) -> bool:
    if dtype != torch.bfloat16 or not WINDOW_ATTENTION_MMA:
        return False
    from . import library
    return bool(library().vlrf_attn_window_mma_takes(n_heads, n_kv_heads, dk, dv, bt, ldq, ld_out))


def attention_window_kind(dtype: torch.dtype, dk: int, dv: int, n_heads: int, n_kv_heads: int) -> dict:
    """Which kernels attention with these sizes runs on."""
    kind = "mma.sync" if _window_mma_takes(dtype, n_heads, n_kv_heads, dk, dv, 64, n_heads * dk, n_heads * dv) else "CUDA cores"
    return {"prompt": kind, "decode": kind}


def window_decode_splits(n_rows: int, n_kv_heads: int, max_context: int, window: int, keep_first: int = 0) -> int:
    """Into how many parts a decode step cuts each context for the tensor-core kernel: parts of at least two key tiles,
    about two CTAs an SM in all."""
    forced = os.environ.get("VLRF_B200_DECODE_SPLITS")
    if forced:
        return max(1, min(16, int(forced)))
    reach = min(max_context, window + 63 + (-(-keep_first // 64)) * 64) if window > 0 else max_context
    tiles = -(-reach // 64)
    # (a part costs a second kernel that merges them: parts only where the step's CTAs would not fill the GPU otherwise)
    return max(1, min(16, tiles // 2, (2 * sm_count()) // max(1, n_rows * n_kv_heads)))


def attention_window_step(q, k_cache, v_cache, block_table, out, ctx, n_heads: int, n_kv_heads: int, dk: int, dv: int, scale: float,
                          window: int, out_scale: float, *, softcap: float = 0.0, keep_first: int = 0, sink=None, gate=None) -> None:
    """The attention of a step (prompt tokens, single tokens or a mix) with the kernel that suits it: bfloat16 sizes that
    the tensor-core kernel takes go there (a decode step's contexts cut into parts), everything else to the kernel
    that takes a warp per token and head."""
    bt = k_cache.shape[2]
    if _window_mma_takes(q.dtype, n_heads, n_kv_heads, dk, dv, bt, q.shape[1], out.stride(0)) and q.data_ptr() % 16 == 0 \
            and out.data_ptr() % 4 == 0:
        _rows(out, "out", q.dtype)
        n_split, partials = 1, None
        if ctx.max_new == 1:
            n_split = window_decode_splits(ctx.n_tokens, n_kv_heads, ctx.max_context, window, keep_first)
            if n_split > 1:
                partials = ctx.ws.get("window_partials", ctx.n_tokens * n_heads * n_split, dv + 2, torch.float32)
        if sink is not None:
            _dev(sink, "sink", torch.float32)
            if sink.numel() != n_heads:
                raise KernelError("attention_window: one sink per query head")
        _check_head_gate(gate, ctx.n_tokens, n_heads)
        call("vlrf_attn_window_mma_ex", _ptr(q), q.shape[1], _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
             _ptr(ctx.seq_slot), _ptr(ctx.seq_start), _ptr(ctx.seq_pos0), _ptr(out), out.stride(0), _ptr(partials), ctx.n_seqs,
             ctx.max_new, n_heads, n_kv_heads, dk, dv, bt, float(scale), int(window), float(out_scale), n_split, float(softcap),
             int(keep_first), _ptr(sink), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(ctx.dev_err), _stream())
        return
    attention_window(q, k_cache, v_cache, block_table, ctx.tok_slot, ctx.tok_pos, out, ctx.n_tokens, n_heads, n_kv_heads, dk, dv,
                     scale, window, out_scale, ctx.dev_err, softcap=softcap, keep_first=keep_first, sink=sink, gate=gate)


def ssd_scan_step(xbc, proj, dt_off: int, dt_bias, a_log, d_skip, state, ctx, y, n_heads: int, n_groups: int, n_state: int, p: int) -> None:
    """The recurrence of a step with the kernel that suits it."""
    ssd_scan(xbc, proj, dt_off, dt_bias, a_log, d_skip, state, ctx.seq_slot, ctx.seq_start, ctx.seq_pos0, y, ctx.n_seqs, n_heads,
             n_groups, n_state, p, ctx.max_new)
