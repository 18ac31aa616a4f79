"""Python faces of the CUDA kernels: each takes torch tensors on the device,
checks what the kernel cannot check itself, and launches on torch's current
stream.  Shapes and dtypes a kernel does not take are refused with an error.
"""
from __future__ import annotations

import math
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .loader import KernelError, check, library, require_cuda
from .profile import enabled as _profiling, region

F32, BF16 = 0, 1


def dtype_code(t) -> int:
    dt = t if isinstance(t, torch.dtype) else t.dtype
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dt} is not taken by the kernels (float32, bfloat16)")


def _p(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream of device 0 as a handle for the launchers (the raw query costs a fraction
    of a microsecond; `torch.cuda.current_stream()` several, once per kernel launch)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(0))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _nb(*ts) -> int:
    """Bytes of the given tensors (what a kernel that touches each once has to move)."""
    return sum(t.numel() * t.element_size() for t in ts if t is not None)


def _dev(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            require_cuda()
            raise KernelError("kernel operands must live on the CUDA device")
        if t is not None and not t.is_contiguous():
            raise KernelError("kernel operands must be contiguous")


_SMS = [0]


def sm_count() -> int:
    """SMs of the device (148 on a B200), asked once: grids and split counts are sized by it."""
    if not _SMS[0]:
        _SMS[0] = int(torch.cuda.get_device_properties(0).multi_processor_count)
    return _SMS[0]


# ---------------------------------------------------------------------------
def embed_gather(ids: torch.Tensor, table: torch.Tensor, err: torch.Tensor,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[t] = float32(table[ids[t]]); an id outside the table sets the error word."""
    _dev(ids, table, err)
    T, (V, D) = ids.shape[0], table.shape
    if out is None:
        out = torch.empty((T, D), dtype=torch.float32, device=table.device)
    lib = library("elementwise.cu")
    with region("embed_gather", T * D * table.element_size() + _nb(out)):
        check(lib.aie_embed_gather(_p(ids), _p(table), c_int(dtype_code(table)), _p(out), c_int(T),
                                   c_int(D), c_int(V), _p(err), _stream()), "embed_gather")
    return out


def take_sampled_ids(ids: torch.Tensor, src: torch.Tensor, last: torch.Tensor, err: torch.Tensor) -> None:
    """ids[t] = last[src[t]] where src[t] >= 0 (int32, in place): tokens that the previous step
    sampled and the host has not read yet."""
    _dev(ids, src, last, err)
    lib = library("elementwise.cu")
    check(lib.aie_take_sampled_ids(_p(ids), _p(src), _p(last), c_int(ids.shape[0]), c_int(last.shape[0]),
                                   _p(err), _stream()), "take_sampled_ids")


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                write_back: bool = True, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """s = x (+ delta); out = (s / sqrt(mean(s^2) + eps)) * weight.  `x` is the
    float32 residual stream and receives s when `write_back`; `rows` picks rows.
    `delta` may be [parts, T, D]: the parts of a split product, added here in order."""
    _dev(x, delta, weight, rows)
    if x.dtype != torch.float32:
        raise KernelError("add_rmsnorm: the residual stream must be float32")
    D = x.shape[-1]
    if weight.shape != (D,):
        raise KernelError(f"add_rmsnorm: weight shape {tuple(weight.shape)} != ({D},)")
    parts, part_stride = 1, 0
    if delta is not None and delta.dim() == 3:        # [parts, T, D]: parts of a split product
        parts, part_stride = delta.shape[0], delta.stride(0)
        if delta.shape[1:] != x.shape:
            raise KernelError("add_rmsnorm: delta parts differ in shape from x")
    elif delta is not None and delta.shape != x.shape:
        raise KernelError("add_rmsnorm: delta shape differs from x")
    n = x.shape[0] if rows is None else rows.shape[0]
    if out is None:
        out = torch.empty((n, D), dtype=out_dtype, device=x.device)
    lib = library("elementwise.cu")
    stored = write_back and rows is None and delta is not None      # without a branch to add, the stream is as it was
    with region("add_rmsnorm", n * D * 4 * (2 if stored else 1) + (_nb(delta) if rows is None else 0) + _nb(out)):
        check(lib.aie_add_rmsnorm(_p(x), _p(delta), c_int(dtype_code(delta) if delta is not None else 0),
                                  _p(weight), c_int(dtype_code(weight)), _p(out),
                                  c_int(dtype_code(out)), _p(rows), c_int(n), c_int(D), c_float(eps),
                                  c_int(1 if stored else 0), c_int(parts),
                                  c_longlong(part_stride), _stream()),
              "add_rmsnorm")
    return out


def silu_mul(gu: torch.Tensor, out: Optional[torch.Tensor] = None, block: int = 0) -> torch.Tensor:
    """a[t, f] = silu(gate) * up.  block == 0: gu[t] = [gate (F) | up (F)]; block > 0: gu[t]
    is in groups of `block` gate columns followed by their `block` up columns."""
    _dev(gu)
    T, F2 = gu.shape
    F = F2 // 2
    if out is None:
        out = torch.empty((T, F), dtype=gu.dtype, device=gu.device)
    lib = library("elementwise.cu")
    with region("silu_mul", _nb(gu, out)):
        check(lib.aie_silu_mul(_p(gu), _p(out), c_int(dtype_code(gu)), c_int(T), c_int(F), c_int(block),
                               _stream()), "silu_mul")
    return out


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if x.dtype == dtype:
        return x
    _dev(x)
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    lib = library("elementwise.cu")
    with region("cast", _nb(x, out)):
        check(lib.aie_cast(_p(x), c_int(dtype_code(x)), _p(out), c_int(dtype_code(out)),
                           c_longlong(x.numel()), _stream()), "cast")
    return out


# ---------------------------------------------------------------------------
def gemm_f32(a: torch.Tensor, w: torch.Tensor, rows: Optional[torch.Tensor] = None,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] = a[M, K] . w[N, K]^T in true float32 (FMA on CUDA cores)."""
    _dev(a, w, rows)
    if a.dtype != torch.float32:
        raise KernelError("gemm_f32: activations must be float32")
    K = a.shape[1]
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm_f32: inner sizes differ ({K} vs {w.shape[1]})")
    M = a.shape[0] if rows is None else rows.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    lib = library("gemm_f32.cu")
    with region("gemm_f32", _nb(w, out) + M * K * 4, 2.0 * M * N * K):
        check(lib.aie_gemm_f32(_p(a), _p(w), c_int(dtype_code(w)), _p(out), _p(rows), c_int(M), c_int(N),
                               c_int(K), c_int(out.stride(0)), _stream()), "gemm_f32")
    return out


def tc_tile(T: int) -> int:
    """Token tile of the tcgen05 product: the smallest of 16 .. 256 that holds T, else 256."""
    for bn in (16, 32, 64, 128, 256):
        if T <= bn:
            return bn
    return 256


def tc_splits(T: int, N: int, K: int, bn: int) -> int:
    """Parts to cut K into.  A weight with fewer 128-row tiles than the machine has SMs is
    cut so that the grid comes close to three CTAs per SM (what fits beside each other with
    4-stage rings), each part at least 12 K blocks of 64: measured inside whole decode steps
    of 1 to 64 tokens, K = 4096 is best cut into 5 parts (fewer leave SMs idle, more pay for
    their unjoined float32 parts, which the consumer reads).  A weight with more tiles is not cut."""
    tiles = ((N + 127) // 128) * ((T + bn - 1) // bn)
    kb = (K + 63) // 64
    if tiles >= sm_count():
        return 1
    return max(1, min((_TC_CTAS_PER_SM * sm_count()) // tiles, kb // _TC_MIN_KB))


# split K: at least this many K blocks of 64 a part, at most this many CTAs an SM.  Swept inside whole decode steps
# of 1, 8 and 64 requests (8B shape): (12, 3) and (12, 2) are equal and best; 8 or 6 blocks a part cost 0-2 %,
# 20 / 32 / 56 blocks a part 2 / 7 / 20 %, four CTAs an SM 4-7 %.
_TC_MIN_KB = 12
_TC_CTAS_PER_SM = 3
TC_SWIGLU_BLOCK = 64     # gate/up rows per half of a 128-row weight tile


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, err: torch.Tensor,
            bn: Optional[int] = None, splits: Optional[int] = None, swiglu: bool = False,
            raw_parts: bool = False):
    """bfloat16 x . w^T on tcgen05 tensor cores fed by TMA; None when the sizes are not
    taken (K not a multiple of 8).  swiglu: w is the fused gate/up weight [2F, K] in tiles
    of 64 gate rows + their 64 up rows; the result is silu(gate) * up, [T, F].
    raw_parts: the parts of a split K are not joined: the result is float32
    [splits, T, N] and whoever reads it adds the parts (the norm and rotary kernels do)."""
    T, K = x.shape
    N = w.shape[0]
    if K % 8 or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or (swiglu and N % 128):
        return None
    _dev(x, w, err)
    bn = bn or tc_tile(T)
    splits = splits or tc_splits(T, N, K, bn)
    if swiglu:
        splits = 1 if raw_parts else min(splits, 8)
    kb = (K + 63) // 64
    splits = max(1, min(splits, kb))
    splits = -(-kb // -(-kb // splits))      # no part without K blocks: 64 blocks in 9 parts of 8 are 8 parts
    if raw_parts and splits > 1:
        out = torch.empty((splits, T, N), dtype=torch.float32, device=x.device)
    else:
        raw_parts = False
        splits = min(splits, 8)              # joined inside a cluster of at most 8 CTAs
        out = torch.empty((T, N // 2 if swiglu else N), dtype=out_dtype, device=x.device)
    lib = library("gemm_tc.cu")
    with region("gemm_tc_swiglu" if swiglu else "gemm_tc", _nb(x, w, out), 2.0 * T * N * K):
        check(lib.aie_gemm_tc(_p(x), _p(w), _p(out), c_int(dtype_code(out)), c_int(T), c_int(N), c_int(K),
                              c_int(out.stride(-2)), c_int(bn), c_int(splits), c_int(1 if swiglu else 0),
                              c_int(1 if raw_parts else 0), _p(err), _stream()), "gemm_tc")
    return out


TC_MAX_TOKENS = 64       # up to here the tcgen05 kernel of this package; above, the library product
TC_ROPE_MAX_TOKENS = 16  # up to here the q/k/v product rotates and writes the cache in its epilogue


def linear_parts(x: torch.Tensor, w: torch.Tensor, err: Optional[torch.Tensor] = None,
                 out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """x . w^T for a consumer that can add parts (the next norm, the rotary kernel): float32
    [parts, T, N] when a small bfloat16 step cut K and left the parts unjoined, else [T, N]
    in `out_dtype`."""
    if (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] <= TC_MAX_TOKENS
            and err is not None):
        y = gemm_tc(x, w, torch.float32, err, raw_parts=True)
        if y is not None:
            return y
    return linear(x, w, out_dtype, err)


def linear_add(stream: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> bool:
    """stream [T, N] float32 += x . w^T in place, the sum taken in float32 inside the library product (its
    epilogue reads the stream and writes it back), for bfloat16 steps of more than 64 tokens: the branch
    output never travels through memory on its own.  False when the step is not of that kind (nothing
    was done): the caller takes `linear_parts` and lets the next norm add."""
    if (x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or stream.dtype != torch.float32
            or x.shape[0] <= TC_MAX_TOKENS or stream.shape != (x.shape[0], w.shape[0]) or not stream.is_contiguous()):
        return False
    _dev(x, w, stream)
    with region("gemm_library", _nb(x, w) + 2 * _nb(stream), 2.0 * x.shape[0] * w.shape[0] * w.shape[1]):
        torch.addmm(stream, x, w.t(), out_dtype=torch.float32, out=stream)
    return True


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           err: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x . w^T.  float32 activations (or a weight stored in 32-bit) take the true
    float32 kernel.  bfloat16 x bfloat16: steps of up to 64 tokens take this package's
    tcgen05 kernel (a weight stream); more tokens take the library matrix product, as the
    reference's engine does for its products
    (crates/ai-engine-candle/src/paged/transformer.rs:153-155)."""
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.float32 or w.dtype == torch.float32:
        y = gemm_f32(cast(x, torch.float32), w)
        return cast(y, out_dtype)
    if x.shape[0] <= TC_MAX_TOKENS and err is not None:
        y = gemm_tc(x, w, out_dtype, err)
        if y is not None:
            return y
    _dev(x, w)
    with region("gemm_library", _nb(x, w) + x.shape[0] * w.shape[0] * (4 if out_dtype == torch.float32 else 2),
                2.0 * x.shape[0] * w.shape[0] * w.shape[1]):
        if out_dtype == torch.float32:
            return torch.mm(x, w.t(), out_dtype=torch.float32)
        return torch.mm(x, w.t())


def linear_swiglu(x: torch.Tensor, w_gu: torch.Tensor, block: int = 0,
                  err: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(x . gate^T) * (x . up^T) for the fused gate/up weight [2F, K]; [T, F] in x's
    dtype.  block == 0: rows [0, F) are gate, [F, 2F) up.  block == 64: tiles of 64 gate
    rows + their 64 up rows, which lets the tcgen05 kernel apply the activation in its
    epilogue when the step is small."""
    if (block == TC_SWIGLU_BLOCK and x.dtype == torch.bfloat16 and w_gu.dtype == torch.bfloat16
            and x.shape[0] <= TC_MAX_TOKENS and err is not None):
        y = gemm_tc(x, w_gu, x.dtype, err, swiglu=True)
        if y is not None:
            return y
    return silu_mul(linear(x, w_gu, x.dtype, err), block=block)


def linear_rope_kv(x: torch.Tensor, w_qkv: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                   positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor,
                   inv_freq: torch.Tensor, H: int, K: int, d: int, err: torch.Tensor,
                   write: bool = True) -> Optional[torch.Tensor]:
    """The q/k/v projection of a small bfloat16 step with the rotation and the cache write in
    its epilogue (one kernel instead of product + rotary kernel); returns q [T, H, d], or None
    when the sizes are not taken: more than 16 tokens, a head size that does not divide 128,
    a partial rotation, K not a multiple of 8."""
    T, Kin = x.shape
    N = w_qkv.shape[0]
    if (T > TC_ROPE_MAX_TOKENS or x.dtype != torch.bfloat16 or w_qkv.dtype != torch.bfloat16
            or k_pages.dtype != torch.bfloat16 or Kin % 8 or d % 2 or 128 % d or N % 128
            or N != (H + 2 * K) * d or inv_freq.shape[0] * 2 != d):
        return None
    _dev(x, w_qkv, k_pages, v_pages, positions, token_req, block_table, inv_freq, err)
    num_pages, Kp, P, dp = k_pages.shape
    if (Kp, dp) != (K, d) or v_pages.shape != k_pages.shape:
        raise KernelError("linear_rope_kv: page shape does not fit (K, d)")
    bn = tc_tile(T)
    kb = (Kin + 63) // 64
    splits = max(1, min(8, kb // 8, (3 * sm_count()) // max(1, N // 128)))
    splits = -(-kb // -(-kb // splits))
    q_out = torch.empty((T, H, d), dtype=torch.bfloat16, device=x.device)
    lib = library("gemm_tc.cu")
    with region("gemm_tc_rope", _nb(x, w_qkv) + T * N * 2, 2.0 * T * N * Kin):
        check(lib.aie_gemm_tc_rope(_p(x), _p(w_qkv), c_int(T), c_int(N), c_int(Kin), c_int(bn), c_int(splits),
                                   _p(q_out), _p(k_pages), _p(v_pages), _p(positions), _p(token_req),
                                   _p(block_table), c_int(block_table.shape[1]), c_int(num_pages), c_int(P),
                                   c_int(H), c_int(K), c_int(d), _p(inv_freq), c_int(1 if write else 0), _p(err),
                                   _stream()), "gemm_tc_rope")
    return q_out


# ---------------------------------------------------------------------------
def rope_kv_write(qkv: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                  positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor,
                  inv_freq: torch.Tensor, H: int, K: int, d: int, err: torch.Tensor,
                  q_out: Optional[torch.Tensor] = None, write: bool = True) -> torch.Tensor:
    """Rotate q and k by position, write k and v to their pages; returns q [T, H, d].
    k_pages / v_pages: [num_pages, K, page, d] of one layer."""
    _dev(qkv, k_pages, v_pages, positions, token_req, block_table, inv_freq, err)
    parts, part_stride = 1, 0
    if qkv.dim() == 3:            # [parts, T, width] float32: parts of a split product, added here
        parts, part_stride = qkv.shape[0], qkv.stride(0)
    T = qkv.shape[-2]
    if qkv.shape[-1] != (H + 2 * K) * d:
        raise KernelError("rope_kv_write: qkv width differs from (H + 2K) * d")
    num_pages, Kp, P, dp = k_pages.shape
    if (Kp, dp) != (K, d) or v_pages.shape != k_pages.shape:
        raise KernelError("rope_kv_write: page shape does not fit (K, d)")
    if qkv.dtype != k_pages.dtype and qkv.dtype != torch.float32:
        raise KernelError("rope_kv_write: qkv must be in the cache's dtype or float32")
    rot = inv_freq.shape[0] * 2
    if q_out is None:
        q_out = torch.empty((T, H, d), dtype=k_pages.dtype, device=qkv.device)
    lib = library("rope_kv.cu")
    with region("rope_kv_write", _nb(qkv) + T * (H + 2 * K) * d * k_pages.element_size()):
        check(lib.aie_rope_kv_write(_p(qkv), c_int(dtype_code(qkv)), c_int(parts), c_longlong(part_stride),
                                    _p(q_out), _p(k_pages), _p(v_pages), c_int(dtype_code(k_pages)),
                                    _p(positions), _p(token_req), _p(block_table),
                                    c_int(block_table.shape[1]), c_int(num_pages), c_int(P), c_int(T),
                                    c_int(H), c_int(K), c_int(d), c_int(rot), _p(inv_freq),
                                    c_int(1 if write else 0), _p(err), _stream()), "rope_kv_write")
    return q_out


def paged_attention_plain(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                          positions: torch.Tensor, token_req: torch.Tensor,
                          block_table: torch.Tensor, scale: float, window: int, err: torch.Tensor,
                          out: Optional[torch.Tensor] = None,
                          token_list: Optional[torch.Tensor] = None, cost=(0.0, 0.0)) -> torch.Tensor:
    """softmax(q.k * scale over keys j <= pos (and j > pos - window)) . v per query
    token and head, keys read through the block table.  q, out: [T, H, d].
    `token_list`: only these tokens are computed (the others' rows of out are left)."""
    _dev(q, k_pages, v_pages, positions, token_req, block_table, err, token_list)
    T, H, d = q.shape
    num_pages, K, P, dp = k_pages.shape
    if dp != d or H % K:
        raise KernelError("paged_attention: head sizes do not fit")
    if d > 256:
        raise KernelError(f"paged_attention: head_dim {d} > 256 is not supported")
    if out is None:
        out = torch.empty_like(q)
    lib = library("attention_plain.cu")
    with region("attention_plain", *cost):
        check(lib.aie_paged_attention_plain(_p(q), _p(k_pages), _p(v_pages), _p(out),
                                            c_int(dtype_code(q)), _p(positions), _p(token_req),
                                            _p(block_table), c_int(block_table.shape[1]),
                                            c_int(num_pages), c_int(P),
                                            c_int(T if token_list is None else token_list.shape[0]),
                                            c_int(H), c_int(K), c_int(d), c_int(window), c_float(scale),
                                            _p(token_list), _p(err), _stream()),
              "paged_attention_plain")
    return out


def decode_splits(n_dec: int, kv_heads: int, group: int, max_keys: int, bt_width: int = 0) -> int:
    """How many parts to cut each decode request's keys into so that the grid fills
    the machine (two CTAs fit on each SM), with parts of at least 128
    keys, and no part spanning more block-table entries than a CTA keeps."""
    ctas = n_dec * kv_heads * ((group + 7) // 8)
    want = max(1, (2 * sm_count()) // ctas)   # rounded down: one full wave, no short second one
    s = max(1, min(want, (max_keys + 127) // 128, 64))
    return max(s, (bt_width + 1999) // 2000)


_DECODE_COUNTERS = {}        # device -> zeroed int32 tickets of the decode kernel (they return to zero)


def _decode_counters(device, n: int):
    t = _DECODE_COUNTERS.get(device)
    if t is None or t.numel() < n:
        t = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)
        _DECODE_COUNTERS[device] = t
    return t


def paged_attention_decode(q, k_pages, v_pages, dec_tokens, positions, token_req, block_table,
                           scale: float, window: int, splits: int, err, out,
                           join_in_kernel: bool = False, cost=(0.0, 0.0)) -> None:
    """bfloat16 split-KV attention for the tokens in `dec_tokens` (requests that bring
    one token).  Head sizes 64 and 128.  Uses scratch for the parts when splits > 1; they are
    joined by a second kernel, or (join_in_kernel) by whichever CTA finishes last — measured
    slightly slower in a decode step, kept for callers that want one launch."""
    _dev(q, k_pages, v_pages, dec_tokens, positions, token_req, block_table, err, out)
    T, H, d = q.shape
    num_pages, K, P, _ = k_pages.shape
    n = dec_tokens.shape[0]
    part_o = part_lse = counters = None
    if splits > 1:
        part_o = torch.empty((n, H, splits, d), dtype=torch.float32, device=q.device)
        part_lse = torch.empty((n, H, splits), dtype=torch.float32, device=q.device)
        if join_in_kernel:
            counters = _decode_counters(q.device, n * K * ((H // K + 7) // 8))
    lib = library("attention_fast.cu")
    with region("attention_decode", *cost):
        check(lib.aie_paged_attention_decode(_p(q), _p(k_pages), _p(v_pages), _p(out), _p(part_o),
                                             _p(part_lse), _p(dec_tokens), c_int(n), _p(positions),
                                             _p(token_req), _p(block_table), c_int(block_table.shape[1]),
                                             c_int(num_pages), c_int(P), c_int(H), c_int(K), c_int(d),
                                             c_int(window), c_float(scale), c_int(splits), _p(counters),
                                             _p(err), _stream()), "paged_attention_decode")


PREFILL_TILE = 128       # query tokens per CTA of the tensor-core attention kernel


def paged_attention_prefill(q, k_pages, v_pages, tiles, q_start, q_len, ctx_len, block_table,
                            scale: float, window: int, err, out, cost=(0.0, 0.0)) -> None:
    """bfloat16 tensor-core attention for requests that bring more than one token.
    `tiles`: int32 [n, 2] = (request row, offset of a PREFILL_TILE-token tile in its tokens).
    Head sizes 64 and 128."""
    _dev(q, k_pages, v_pages, tiles, q_start, q_len, ctx_len, block_table, err, out)
    T, H, d = q.shape
    num_pages, K, P, _ = k_pages.shape
    lib = library("attention_fast.cu")
    with region("attention_prefill_mma", *cost):
        check(lib.aie_paged_attention_prefill(_p(q), _p(k_pages), _p(v_pages), _p(out), _p(tiles),
                                              c_int(tiles.shape[0]), _p(q_start), _p(q_len), _p(ctx_len),
                                              _p(block_table), c_int(block_table.shape[1]),
                                              c_int(num_pages), c_int(P), c_int(H), c_int(K), c_int(d),
                                              c_int(window), c_float(scale), _p(err), _stream()),
              "paged_attention_prefill")


def paged_attention_prefill_tc(q, k_pages, v_pages, tiles, q_start, q_len, ctx_len, block_table,
                               scale: float, window: int, err, out, cost=(0.0, 0.0), pair: bool = False) -> bool:
    """The tcgen05 version of paged_attention_prefill (scores and outputs in tensor memory,
    operands by TMA).  Takes head sizes 64 and 128, pages of 8 .. 128 keys that divide 128, no window; returns
    False when it does not take the sizes (nothing was launched).  `pair`: the kernel whose CTAs take two tiles
    each; `tiles` then lists units of 2 * PREFILL_TILE tokens (request row, offset of the unit)."""
    _dev(q, k_pages, v_pages, tiles, q_start, q_len, ctx_len, block_table, err, out)
    T, H, d = q.shape
    num_pages, K, P, _ = k_pages.shape
    if d not in (64, 128) or window > 0 or P < 8 or P > 128 or 128 % P:
        return False
    lib = library("attention_prefill_tc.cu")
    fn = lib.aie_paged_attention_prefill_tc_pair if pair else lib.aie_paged_attention_prefill_tc
    with region("attention_prefill_tcgen05", *cost):
        rc = fn(_p(q), _p(k_pages), _p(v_pages), _p(out), _p(tiles), c_int(tiles.shape[0]), _p(q_start), _p(q_len),
                _p(ctx_len), _p(block_table), c_int(block_table.shape[1]), c_int(num_pages), c_int(P), c_int(T),
                c_int(H), c_int(K), c_int(d), c_int(window), c_float(scale), _p(err), _stream())
    if rc == -2:
        return False
    check(rc, "paged_attention_prefill_tc")
    return True


def prefill_takes_pairs(n_tiles: int, n_units: int, heads: int) -> bool:
    """Whether the tcgen05 prompt kernel with two query tiles per CTA is the faster one for a step with `n_tiles`
    tiles in `n_units` units of two.  Measured on heads of 128 and of 64: it takes 0.80-0.86 of the one-tile
    kernel's time when nearly all units are whole and its CTAs (units x heads) fill the SMs in whole rounds about as
    well as the one-tile kernel's; with a lone tile in a unit it runs at half speed, and with fewer CTAs than SMs
    the longest CTA decides, which is twice as long."""
    if n_units == 0 or n_tiles < 1.8 * n_units:
        return False
    sms = sm_count()
    w1, w2 = n_tiles * heads / sms, n_units * heads / sms
    if w2 <= 1.0:
        return False
    return 0.86 * math.ceil(w2) / w2 < math.ceil(w1) / w1


def paged_attention(q, k_pages, v_pages, ctx, work, block_table, scale: float, window: int):
    """Attention of a step's query tokens over the cache.  `ctx` gives the step's generic arrays
    (positions, token_req, q_start, q_len, ctx_len, R), `work` the attention work lists derived from
    them (decode_tokens, prefill_tiles, n_decode, max_decode_len).  float32 takes the plain
    kernel.  bfloat16 with a head size of 64 or 128: requests that bring one token
    take the split-KV decode kernel, the others a tensor-core kernel for portions of
    prompts (tcgen05 for head size 128 without a window, else mma.sync); other head sizes
    take the plain kernel."""
    T, H, d = q.shape
    K = k_pages.shape[1]
    fast = q.dtype == torch.bfloat16 and d in (64, 128)
    dec_cost = pre_cost = (0.0, 0.0)
    if _profiling() and hasattr(ctx, "h_q_len"):      # keys read and products done, from the host's lengths
        ql, cl = ctx.h_q_len.astype(float), ctx.h_ctx_len.astype(float)
        if window > 0:
            cl = cl.clip(max=float(window))
        es = k_pages.element_size()
        lone = ql == 1
        keys = float((cl[lone] + 1).sum())
        dec_cost = (keys * K * d * 2 * es, 4.0 * keys * H * d)
        pairs = float((ql[~lone] * cl[~lone] + ql[~lone] * (ql[~lone] + 1) / 2).sum())
        pre_cost = (float((cl[~lone] + ql[~lone]).sum()) * K * d * 2 * es + float(ql[~lone].sum()) * H * d * 2 * es,
                    4.0 * pairs * H * d)
    if not fast:
        return paged_attention_plain(q, k_pages, v_pages, ctx.positions, ctx.token_req, block_table,
                                     scale, window, ctx.err,
                                     cost=(dec_cost[0] + pre_cost[0], dec_cost[1] + pre_cost[1]))
    out = torch.empty_like(q)
    if work.n_decode:
        keys = work.max_decode_len if window <= 0 else min(window, work.max_decode_len)
        paged_attention_decode(q, k_pages, v_pages, work.decode_tokens, ctx.positions, ctx.token_req,
                               block_table, scale, window,
                               decode_splits(work.n_decode, K, H // K, keys, block_table.shape[1]),
                               ctx.err, out, cost=dec_cost)
    if work.n_decode < ctx.R:
        pairs = getattr(work, "prefill_pairs", None)
        if pairs is not None and prefill_takes_pairs(work.prefill_tiles.shape[0], pairs.shape[0], H):
            took = paged_attention_prefill_tc(q, k_pages, v_pages, pairs, ctx.q_start, ctx.q_len, ctx.ctx_len,
                                              block_table, scale, window, ctx.err, out, cost=pre_cost, pair=True)
        else:
            took = paged_attention_prefill_tc(q, k_pages, v_pages, work.prefill_tiles, ctx.q_start, ctx.q_len,
                                              ctx.ctx_len, block_table, scale, window, ctx.err, out, cost=pre_cost)
        if not took:
            paged_attention_prefill(q, k_pages, v_pages, work.prefill_tiles, ctx.q_start, ctx.q_len,
                                    ctx.ctx_len, block_table, scale, window, ctx.err, out, cost=pre_cost)
    return out
