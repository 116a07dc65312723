"""Python face of the CUDA library: one function per launcher, taking torch tensors.

There is no CPU fallback and no other implementation behind these names: if the
library cannot be built or loaded, importing a function's first use raises.  All
launches go to torch's current CUDA stream, so they can be captured in a graph.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    """A launcher refused its arguments or CUDA reported an error."""


_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        path = build.ensure_built()
        try:
            handle = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the CUDA library {path}: {e}") from None
        handle.gg_last_error.restype = ctypes.c_char_p
        _LIB = handle
    return _LIB


def library_file() -> str:
    lib()
    return build.library_path()


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream of the current device as a pointer (asked on every launch: a graph
    capture runs on a stream of its own).  The raw accessor costs a tenth of building a
    torch.cuda.Stream object, which matters at a few hundred launches per prompt step."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


launches = 0          # kernels of this library launched by this process (a captured graph counts once)


def _check(rc: int, n: int = 1) -> None:
    global launches
    if rc != 0:
        raise KernelError(lib().gg_last_error().decode())
    launches += n


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dt}")


def _cuda(*tensors):
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise KernelError("kernel arguments must be contiguous CUDA tensors")


def device_capability() -> int:
    return int(lib().gg_device_capability())


def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
                 bad_id: Optional[torch.Tensor] = None, token_src: Optional[torch.Tensor] = None,
                 prev_tokens: Optional[torch.Tensor] = None) -> None:
    """out[t, :] = float32(table[id_t, :]); ids int32 [T], out float32 [T, H].  Where
    token_src[t] >= 0 the id is prev_tokens[token_src[t]] (a token still on the device)."""
    _cuda(ids, table, out, token_src, prev_tokens)
    T, (V, H) = ids.numel(), table.shape
    if out.dtype != torch.float32 or out.shape[-1] != H or ids.dtype != torch.int32:
        raise KernelError("embed_gather: out must be float32 [T, H], ids int32")
    _check(lib().gg_embed_gather(_p(ids), _p(table), dtype_code(table.dtype), _p(out),
                                 T, H, V, _p(bad_id), _p(token_src), _p(prev_tokens), _stream()))


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None,
                write_back: bool = True) -> None:
    """x = resid[r] (+ delta[r]); resid[r] = x if write_back; out[i] = rmsnorm(x) * weight,
    r = rows[i] if rows is given else i.  resid float32, weight float32, out/delta same dtype.
    ``rows`` and ``weight`` are read before the kernel ahead of this one has finished: they must
    not be that kernel's output (the engine gives the step's packed row list)."""
    _cuda(resid, delta, weight, out, rows)
    H = resid.shape[-1]
    n = rows.numel() if rows is not None else out.shape[0]
    if resid.dtype != torch.float32 or weight.dtype != torch.float32 or weight.numel() != H:
        raise KernelError("add_rmsnorm: residual and weight must be float32 of one width")
    if delta is not None and delta.dtype != out.dtype:
        raise KernelError("add_rmsnorm: delta and out differ in dtype")
    _check(lib().gg_add_rmsnorm(_p(resid), _p(delta), _p(weight), _p(out), dtype_code(out.dtype),
                                _p(rows), n, H, ctypes.c_float(eps), int(write_back), _stream()))


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _cuda(gate_up, out)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I) or gate_up.dtype != out.dtype:
        raise KernelError("silu_mul: input must be [T, 2I] of the output's dtype")
    _check(lib().gg_silu_mul(_p(gate_up), _p(out), dtype_code(out.dtype), T, I, _stream()))


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, slot_mapping: Optional[torch.Tensor],
                  inv_freq: Optional[torch.Tensor], kcache: Optional[torch.Tensor],
                  vcache: Optional[torch.Tensor], nh: int, nkv: int, d: int, page_size: int,
                  interleaved: bool = False, write_cache: bool = True) -> None:
    """Rotate q and k heads of qkv [T, (nh+2nkv)*d] in place and scatter k, v into the
    paged cache [pages, nkv, page_size, d] at slot_mapping[t].  ``positions``, ``slot_mapping``
    and ``inv_freq`` are read before the kernel ahead of this one has finished: they must not be
    that kernel's output (the engine gives the step's packed lists)."""
    _cuda(qkv, positions, slot_mapping, inv_freq, kcache, vcache)
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * d:
        raise KernelError("rope_kv_write: qkv width is not (nh + 2 nkv) * d")
    if inv_freq is not None and inv_freq.dtype != torch.float64:
        raise KernelError("rope_kv_write: inverse frequencies must be float64")
    if kcache is not None and kcache.dtype != qkv.dtype:
        raise KernelError("rope_kv_write: cache and activations differ in dtype")
    rot = 2 * inv_freq.numel() if inv_freq is not None else 0
    _check(lib().gg_rope_kv_write(_p(qkv), dtype_code(qkv.dtype), _p(positions), _p(slot_mapping),
                                  _p(inv_freq), _p(kcache), _p(vcache), T, nh, nkv, d, rot,
                                  page_size, int(interleaved), int(write_cache), _stream()))


def attn_prefill(q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                 block_tables: torch.Tensor, bt_stride: int, cu_q_lens: torch.Tensor,
                 context_lens: torch.Tensor, tile_seq: torch.Tensor, tile_q0: torch.Tensor,
                 num_tiles: int, out: torch.Tensor, nh: int, nkv: int, d: int, page_size: int,
                 window: int, scale: float, tile64_seq: Optional[torch.Tensor] = None,
                 tile64_q0: Optional[torch.Tensor] = None, num_tiles64: int = 0,
                 allow_mma: bool = True, tile128_seq: Optional[torch.Tensor] = None,
                 tile128_q0: Optional[torch.Tensor] = None, num_tiles128: int = 0,
                 allow_tc: bool = True) -> None:
    """Causal attention of prompt portions over the paged cache.  ``tile_*`` list tiles
    of 16 queries (general kernel), ``tile64_*`` of 64 (mma.sync kernel: bfloat16, head
    size 64 or 128), ``tile128_*`` of 128 (tcgen05 kernel: bfloat16, head size 64 or 128); the
    most specialised kernel whose list is given and that is allowed runs.  ``allow_tc``: 2 =
    only the tcgen05 kernel with one head per CTA, not the one with two heads of a kv head."""
    global tc_launched
    use_tc = allow_tc and tile128_seq is not None and kcache.dtype == torch.bfloat16 and d in (64, 128)
    if use_tc:
        tc_launched = True
    _check(lib().gg_attn_prefill(_p(q), ctypes.c_longlong(q_stride), _p(kcache), _p(vcache),
                                 dtype_code(kcache.dtype), _p(block_tables), bt_stride,
                                 _p(cu_q_lens), _p(context_lens), _p(tile_seq), _p(tile_q0),
                                 num_tiles, _p(tile64_seq), _p(tile64_q0), num_tiles64,
                                 _p(tile128_seq), _p(tile128_q0), num_tiles128, _p(out),
                                 q.shape[0], kcache.shape[0], nh, nkv, d, page_size, window,
                                 ctypes.c_float(scale), int(allow_mma), int(allow_tc),
                                 _p(tc_status(q.device)) if use_tc else ctypes.c_void_p(0), _stream()))


def attn_decode(q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                block_tables: torch.Tensor, bt_stride: int, cu_q_lens: torch.Tensor,
                context_lens: torch.Tensor, dec_seqs: torch.Tensor, n_dec: int, num_splits: int,
                part_o: torch.Tensor, part_ml: torch.Tensor, out: torch.Tensor, nh: int, nkv: int,
                d: int, page_size: int, window: int, scale: float, allow_mma: bool = True) -> None:
    """Attention of single decoded tokens, split over the context and merged."""
    if part_o.numel() < n_dec * nh * num_splits * d or part_ml.numel() < n_dec * nh * num_splits * 2:
        raise KernelError("attn_decode: scratch too small")
    _check(lib().gg_attn_decode(_p(q), ctypes.c_longlong(q_stride), _p(kcache), _p(vcache),
                                dtype_code(kcache.dtype), _p(block_tables), bt_stride,
                                _p(cu_q_lens), _p(context_lens), _p(dec_seqs), n_dec, num_splits,
                                _p(part_o), _p(part_ml), _p(out), nh, nkv, d, page_size, window,
                                ctypes.c_float(scale), int(allow_mma), _stream()), 2)


def attn_decode_rope_ok(dtype: torch.dtype, nh: int, nkv: int, d: int, inv_freq: Optional[torch.Tensor],
                        interleaved: bool) -> bool:
    """Whether attn_decode_rope takes this shape: bfloat16, head size 64 or 128, at most 16
    heads per kv head, half-split rotation over the whole head."""
    return (dtype == torch.bfloat16 and d in (64, 128) and nh // nkv <= 16 and inv_freq is not None
            and inv_freq.dtype == torch.float64 and 2 * inv_freq.numel() == d and not interleaved)


def attn_decode_rope(qkv: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                     block_tables: torch.Tensor, bt_stride: int, cu_q_lens: torch.Tensor,
                     context_lens: torch.Tensor, dec_seqs: torch.Tensor, n_dec: int, num_splits: int,
                     part_o: torch.Tensor, part_ml: torch.Tensor, out: torch.Tensor, nh: int, nkv: int,
                     d: int, page_size: int, window: int, scale: float, positions: torch.Tensor,
                     slot_mapping: Optional[torch.Tensor], inv_freq: torch.Tensor,
                     write_cache: bool = True) -> None:
    """rope_kv_write and attn_decode of single decoded tokens in one kernel: qkv is the raw
    projection output and stays as it is; k (rotated) and v land in the cache."""
    _cuda(qkv, positions, slot_mapping, inv_freq, kcache, vcache)
    if not attn_decode_rope_ok(qkv.dtype, nh, nkv, d, inv_freq, False) or kcache.dtype != qkv.dtype:
        raise KernelError("attn_decode_rope: shape or dtype not taken (see attn_decode_rope_ok)")
    if qkv.shape[1] != (nh + 2 * nkv) * d or qkv.stride(0) != qkv.shape[1]:
        raise KernelError("attn_decode_rope: qkv must be contiguous [T, (nh + 2 nkv) * d]")
    if part_o.numel() < n_dec * nh * num_splits * d or part_ml.numel() < n_dec * nh * num_splits * 2:
        raise KernelError("attn_decode_rope: scratch too small")
    if write_cache and slot_mapping is None:
        raise KernelError("attn_decode_rope: cache write without slots")
    _check(lib().gg_attn_decode_rope(_p(qkv), ctypes.c_longlong(qkv.shape[1]), _p(kcache), _p(vcache),
                                     dtype_code(kcache.dtype), _p(block_tables), bt_stride,
                                     _p(cu_q_lens), _p(context_lens), _p(dec_seqs), n_dec, num_splits,
                                     _p(part_o), _p(part_ml), _p(out), nh, nkv, d, page_size, window,
                                     ctypes.c_float(scale), _p(positions), _p(slot_mapping), _p(inv_freq),
                                     int(write_cache), _stream()), 2)


ATTN_FLAT_MAX_SEQS = 1024   # decoded tokens attn_decode_flat takes in one launch (FLAT_MAX_SEQS in attention_mma.cu)


def attn_prefill_choice(dtype: torch.dtype, d: int, page_size: int, nh: int, nkv: int) -> int:
    """Which tcgen05 prompt kernel attn_prefill(allow_tc=True) runs for a shape on this build and
    device: 3 = two heads per CTA in steps of 128 keys, 2 = the same in steps of 64, 1 = one head
    per CTA, 0 = none."""
    return int(lib().gg_attn_prefill_choice(dtype_code(dtype), d, page_size, nh, nkv))


def attn_decode_flat_ctas(d: int) -> int:
    """CTAs that attn_decode_flat launches for head size d (for sizing its scratch)."""
    return int(lib().gg_attn_decode_flat_ctas(d))


def attn_decode_flat_pieces(n_dec: int, nh: int, nkv: int, d: int) -> int:
    """Partial results attn_decode_flat may leave: scratch part_o holds pieces * 16 * d floats,
    part_ml pieces * 16 * 2."""
    return n_dec * nkv * -(-(nh // nkv) // 16) + attn_decode_flat_ctas(d)


def attn_decode_flat_prefix_ints(n_dec: int, nh: int, nkv: int) -> int:
    """int32 scratch of attn_decode_flat: the tiles before each token, then for each (kv head
    chunk, token) pair the CTAs that hold its first and last piece."""
    return n_dec + 1 + 2 * n_dec * nkv * -(-(nh // nkv) // 16)


def attn_decode_flat(q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                     block_tables: torch.Tensor, bt_stride: int, cu_q_lens: torch.Tensor,
                     context_lens: torch.Tensor, dec_seqs: torch.Tensor, n_dec: int,
                     part_o: torch.Tensor, part_ml: torch.Tensor, prefix: torch.Tensor, out: torch.Tensor,
                     nh: int, nkv: int, d: int, page_size: int, window: int, scale: float) -> None:
    """Attention of single decoded tokens for large batches (bfloat16, head size 64 or 128):
    the 64-key tiles of all (token, kv head) pairs are cut into equal ranges, one per CTA,
    and merged by a second kernel.  ``prefix``: int32 scratch of attn_decode_flat_prefix_ints()."""
    pieces = attn_decode_flat_pieces(n_dec, nh, nkv, d)
    if part_o.numel() < pieces * 16 * d or part_ml.numel() < pieces * 16 * 2 \
            or prefix.numel() < attn_decode_flat_prefix_ints(n_dec, nh, nkv):
        raise KernelError("attn_decode_flat: scratch too small")
    if prefix.dtype != torch.int32 or part_o.dtype != torch.float32 or part_ml.dtype != torch.float32:
        raise KernelError("attn_decode_flat: scratch of the wrong type")
    _check(lib().gg_attn_decode_flat(_p(q), ctypes.c_longlong(q_stride), _p(kcache), _p(vcache),
                                     dtype_code(kcache.dtype), _p(block_tables), bt_stride,
                                     _p(cu_q_lens), _p(context_lens), _p(dec_seqs), n_dec,
                                     _p(part_o), _p(part_ml), _p(prefix), prefix.numel(), _p(out), nh, nkv, d, page_size,
                                     window, ctypes.c_float(scale), _stream()), 2)


ATTN_MAX_CLUSTER = 8  # largest count of slices that the decode kernel merges inside a cluster


def attn_decode_cluster_capacity(dtype: torch.dtype, d: int, splits: int, group: int) -> int:
    """Clusters of `splits` decode CTAs the device holds at once, with `group` query heads
    to a kv head; 0 where attn_decode merges with a kernel of its own instead."""
    if dtype not in (torch.bfloat16, torch.float32):
        return 0
    return int(lib().gg_attn_decode_cluster_capacity(dtype_code(dtype), d, splits, group))


SMALL_M = 16          # most tokens gemm_small_m takes


def small_m_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether out = x @ w^T can go through gemm_small_m."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda
            and 0 < x.shape[0] <= SMALL_M and x.shape[1] % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.is_contiguous())


def gemm_small_m(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False,
                 in_partials: Optional[torch.Tensor] = None, hidden: int = 0, eps: float = 0.0,
                 resid: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None,
                 out_partials: Optional[torch.Tensor] = None) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T for M <= 16 (bfloat16 in, float32 accumulate); out is
    bfloat16 or float32.  ``gated``: w is [2N, K] (gate rows, then up rows) and
    out = silu(x Wg^T) * (x Wu^T) in bfloat16.

    RMSNorm folded in on either side (rms_t = sqrt(mean_k h[t, k]^2 + eps)):
    ``resid``, ``norm_w``, ``out_partials``: the product is added to the float32 residual
    stream ``resid`` [M, N] in place, ``out`` (bfloat16) becomes resid * norm_w, and
    out_partials [ceil(N / 16), 16] float32 gets the sums of resid^2 over each 16 columns.
    ``in_partials`` (+ ``hidden``, ``eps``): x is such an unnormalised resid * norm_w and
    in_partials its partial sums; row t of the result is divided by rms_t."""
    M, K = x.shape
    N = out.shape[1]
    if w.shape != ((2 * N, K) if gated else (N, K)) or out.shape[0] != M or not out.is_contiguous():
        raise KernelError("gemm_small_m: shapes do not fit")
    if gated:
        if out.dtype != torch.bfloat16:
            raise KernelError("gemm_small_m: the gated product writes bfloat16")
        mode = 2
    else:
        mode = 1 if out.dtype == torch.float32 else 0
        if out.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError("gemm_small_m: out must be bfloat16 or float32")
    in_tiles = 0
    if in_partials is not None:
        if in_partials.dtype != torch.float32 or in_partials.dim() != 2 or in_partials.shape[1] != 16 \
                or not in_partials.is_contiguous() or hidden <= 0:
            raise KernelError("gemm_small_m: in_partials must be contiguous float32 [tiles, 16] with the hidden size given")
        in_tiles = in_partials.shape[0]
    if resid is not None or norm_w is not None or out_partials is not None:
        if gated or out.dtype != torch.bfloat16:
            raise KernelError("gemm_small_m: the residual epilogue writes bfloat16 and is not gated")
        if resid is None or norm_w is None or out_partials is None:
            raise KernelError("gemm_small_m: resid, norm_w and out_partials go together")
        if resid.dtype != torch.float32 or resid.shape != (M, N) or not resid.is_contiguous():
            raise KernelError("gemm_small_m: resid must be contiguous float32 [M, N]")
        if norm_w.dtype != torch.float32 or norm_w.numel() != N or not norm_w.is_contiguous():
            raise KernelError("gemm_small_m: norm_w must be contiguous float32 [N]")
        if out_partials.dtype != torch.float32 or not out_partials.is_contiguous() \
                or out_partials.numel() < -(-N // 16) * 16:
            raise KernelError("gemm_small_m: out_partials must be contiguous float32 [ceil(N / 16), 16]")
        mode = 3
    _cuda(w, out, in_partials, resid, norm_w, out_partials)
    _check(lib().gg_gemm_small_m_fused(_p(x), ctypes.c_longlong(x.stride(0)), _p(w), _p(out), M, N, K, mode,
                                       _p(in_partials), in_tiles, int(hidden), ctypes.c_float(eps),
                                       _p(resid), _p(norm_w), _p(out_partials), _stream()))


def gemm_small_m_clamped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, limit: float, alpha: float,
                         shift: float) -> None:
    """The gated product of gemm_small_m (w [2N, K]: gate rows, then up rows) with the clamped
    activation in its epilogue: out = g * sigmoid(alpha * g) * (u + shift), g = min(gate, limit),
    u = clamp(up, -limit, limit); bfloat16, M <= 16."""
    M, K = x.shape
    N = out.shape[1]
    if w.shape != (2 * N, K) or out.shape[0] != M or not out.is_contiguous() or out.dtype != torch.bfloat16:
        raise KernelError("gemm_small_m_clamped: shapes do not fit")
    _cuda(w, out)
    _check(lib().gg_gemm_small_m_clamped(_p(x), ctypes.c_longlong(x.stride(0)), _p(w), _p(out), M, N, K,
                                         ctypes.c_float(limit), ctypes.c_float(alpha), ctypes.c_float(shift), _stream()))


_TC_STATUS = {}
tc_launched = False       # a tcgen05 product was launched since the status word was last checked


def tc_status(device) -> torch.Tensor:
    """The status word gemm_tc writes when one of its bounded waits runs out (0 = fine)."""
    key = torch.device(device).index or 0
    if key not in _TC_STATUS:
        _TC_STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _TC_STATUS[key]


def check_tc_status(device) -> None:
    """Raise if a tensor-core product gave up on a wait since the last check (synchronises)."""
    st = tc_status(device)
    code = int(st.item())
    if code:
        st.zero_()
        raise KernelError(f"gemm_tc gave up waiting on a barrier (code {code}); its output is not valid")


def tc_ok(x: torch.Tensor, w: torch.Tensor, out_cols: int) -> bool:
    """Whether out = x @ w^T can go through gemm_tc."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda and x.shape[0] > 0
            and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and w.is_contiguous()
            and out_cols % 2 == 0)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False,
            pair: bool = False) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T on tcgen05 (bfloat16 in, float32 accumulate in tensor
    memory); out bfloat16 or float32.  ``gated``: w is [2N, K] (gate rows, then up rows) and
    out = silu(x Wg^T) * (x Wu^T) in bfloat16.  ``pair``: the kernel in which two CTAs on two
    SMs share a 256 x 256 tile (cta_group::2)."""
    M, K = x.shape
    N = out.shape[1]
    if w.shape != ((2 * N, K) if gated else (N, K)) or out.shape[0] != M or not out.is_contiguous():
        raise KernelError("gemm_tc: shapes do not fit")
    if gated and out.dtype != torch.bfloat16:
        raise KernelError("gemm_tc: the gated product writes bfloat16")
    if out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError("gemm_tc: out must be bfloat16 or float32")
    mode = 2 if gated else (1 if out.dtype == torch.float32 else 0)
    global tc_launched
    tc_launched = True
    fn = lib().gg_gemm_tc2 if pair else lib().gg_gemm_tc
    _check(fn(_p(x), ctypes.c_longlong(x.stride(0)), _p(w), _p(out), M, N, K, mode,
              _p(tc_status(x.device)), _stream()))


MID_M = 64            # most tokens gemm_mid_m takes


def mid_m_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether out = x @ w^T can go through gemm_mid_m."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda
            and 0 < x.shape[0] <= MID_M and x.shape[1] % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.is_contiguous())


_MID_M_PLANS = {}


def mid_m_plan(M: int, N: int, K: int, gated: bool, device=None):
    """How gemm_mid_m cuts out[M, N] = x[M, K] @ w^T on the current device: (S, boxes, box_rows,
    slabs, ctas_per_sm, ctas_at_once).  It launches S * slabs CTAs."""
    key = (torch.device(device).index if device is not None else torch.cuda.current_device(), M <= 32, N, K, gated)
    plan = _MID_M_PLANS.get(key)
    if plan is None:
        buf = (ctypes.c_int * 6)()
        with torch.cuda.device(key[0]):
            _check(lib().gg_gemm_mid_m_plan(M, N, K, 2 if gated else 0, buf))
        plan = _MID_M_PLANS[key] = tuple(buf)
    return plan


def gemm_mid_m(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T for M <= 64 on tcgen05 with the operands swapped (rows
    of w on the M side of the instruction, tokens on its N side), the rows of w cut into slabs
    so that the CTAs fill the machine evenly, and K split over a thread-block cluster where the
    slabs are few; out bfloat16 or float32.  ``gated``: w is [2N, K] (gate rows, then up rows)
    and out = silu(x Wg^T) * (x Wu^T) in bfloat16."""
    M, K = x.shape
    N = out.shape[1]
    if w.shape != ((2 * N, K) if gated else (N, K)) or out.shape[0] != M or not out.is_contiguous():
        raise KernelError("gemm_mid_m: shapes do not fit")
    if gated and out.dtype != torch.bfloat16:
        raise KernelError("gemm_mid_m: the gated product writes bfloat16")
    if out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError("gemm_mid_m: out must be bfloat16 or float32")
    mode = 2 if gated else (1 if out.dtype == torch.float32 else 0)
    global tc_launched
    tc_launched = True
    _check(lib().gg_gemm_mid_m(_p(x), ctypes.c_longlong(x.stride(0)), _p(w), _p(out), M, N, K, mode,
                               _p(tc_status(x.device)), _stream()))


def gemm_tc_withheld(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """Self-test of gemm_tc's bounded waits: launches it with its loads withheld.  The kernel
    gives up after about a second, sets the status word and returns (check_tc_status raises)."""
    M, K = x.shape
    global tc_launched
    tc_launched = True
    _check(lib().gg_gemm_tc_withheld(_p(x), ctypes.c_longlong(x.stride(0)), _p(w), _p(out), M, out.shape[1], K,
                                     _p(tc_status(x.device)), _stream()))


def pack_decode_step(host, offsets, G: int, B: int, Bp: int, used: int, page_size: int, tokens, token_src,
                     state_slots, context_after, tables) -> None:
    """Fill the packed int32 step buffer ``host`` (a numpy view) for a step of single decoded
    tokens: native code over flat numpy arrays (csrc/host_pack.cu).  ``offsets``: int32 array
    of the buffer's array offsets, ``tables``: per group the cache manager's [state slot,
    logical page] int32 table."""
    import numpy as np
    for a in (host, offsets, tokens, token_src, state_slots, context_after, *tables):
        if a.dtype != np.int32 or not a.flags["C_CONTIGUOUS"]:
            raise KernelError("pack_decode_step: arguments must be contiguous int32 arrays")
    ptrs = (ctypes.c_void_p * max(G, 1))(*[t.ctypes.data for t in tables])
    widths = (ctypes.c_int * max(G, 1))(*[t.shape[1] for t in tables])
    vp = lambda a: ctypes.c_void_p(a.ctypes.data)
    _check(lib().gg_pack_decode_step(vp(host), vp(offsets), G, B, Bp, used, page_size, vp(tokens), vp(token_src),
                                     vp(state_slots), vp(context_after), ptrs, widths), 0)


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = first index of the maximum of logits[r, :] (float32 [R, V])."""
    _cuda(logits, out)
    R, V = logits.shape
    if logits.dtype != torch.float32 or out.dtype != torch.int32:
        raise KernelError("argmax: logits float32, out int32")
    _check(lib().gg_argmax(_p(logits), R, V, _p(out), _stream()))


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: Optional[torch.Tensor],
           top_p: Optional[torch.Tensor], seeds: torch.Tensor, draw_index: torch.Tensor,
           out: torch.Tensor) -> None:
    """Per row: greedy if temperature <= 1e-9, else top-k / top-p / seeded categorical."""
    _cuda(logits, temperature, top_k, top_p, seeds, draw_index, out)
    R, V = logits.shape
    if logits.dtype != torch.float32 or out.dtype != torch.int32 or temperature.dtype != torch.float32:
        raise KernelError("sample: logits/temperature float32, out int32")
    if seeds.dtype != torch.int64 or draw_index.dtype != torch.int64:
        raise KernelError("sample: seeds and draw indices must be int64")
    _check(lib().gg_sample(_p(logits), R, V, _p(temperature), _p(top_k), _p(top_p), _p(seeds),
                           _p(draw_index), _p(out), _stream()))


# ---------------------------------------------------------------- norms with mean and bias, norms on a sublayer's output
def add_norm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
             bias: Optional[torch.Tensor], out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None,
             write_back: bool = True, layer: bool = True) -> None:
    """x = resid[r] (+ delta[r]); out[i] = norm(x), r = rows[i] if rows is given else i.
    ``layer``: (x - mean) / sqrt(var + eps) * weight + bias; else x / sqrt(mean(x^2) + eps) * weight."""
    _cuda(resid, delta, weight, bias, out, rows)
    H = resid.shape[-1]
    n = rows.numel() if rows is not None else out.shape[0]
    if resid.dtype != torch.float32 or weight.dtype != torch.float32 or weight.numel() != H \
            or (bias is not None and (bias.dtype != torch.float32 or bias.numel() != H)):
        raise KernelError("add_norm: residual, weight and bias must be float32 of one width")
    if delta is not None and delta.dtype != out.dtype:
        raise KernelError("add_norm: delta and out differ in dtype")
    _check(lib().gg_add_norm(_p(resid), _p(delta), _p(weight), _p(bias), _p(out), dtype_code(out.dtype), _p(rows),
                             n, H, ctypes.c_float(eps), int(write_back), int(layer), _stream()))


def norm_scale_add(resid: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                   scale: Optional[torch.Tensor], copy: Optional[torch.Tensor], eps: float, layer: bool = True) -> None:
    """resid[t] += scale * norm(y[t]) (scale per channel, or none); copy[t] = resid[t] rounded to
    copy's dtype, if given.  resid float32 [T, H]; y and copy of one dtype."""
    _cuda(resid, y, weight, bias, scale, copy)
    T, H = y.shape
    if resid.dtype != torch.float32 or resid.shape[-1] != H or weight.dtype != torch.float32 or weight.numel() != H:
        raise KernelError("norm_scale_add: residual and weight must be float32 of the input's width")
    for v in (bias, scale):
        if v is not None and (v.dtype != torch.float32 or v.numel() != H):
            raise KernelError("norm_scale_add: bias and scale must be float32 of the input's width")
    if copy is not None and (copy.dtype != y.dtype or copy.shape != y.shape):
        raise KernelError("norm_scale_add: the copy has the input's shape and dtype")
    _check(lib().gg_norm_scale_add(_p(resid), _p(y), _p(weight), _p(bias), _p(scale), _p(copy), dtype_code(y.dtype),
                                   T, H, ctypes.c_float(eps), int(layer), _stream()))


def cast_rows(resid: torch.Tensor, copy: torch.Tensor) -> None:
    """copy = resid rounded to copy's dtype (float32 [T, H] in)."""
    _cuda(resid, copy)
    if resid.dtype != torch.float32 or resid.numel() != copy.numel():
        raise KernelError("cast_rows: float32 in, as many elements out")
    _check(lib().gg_cast_rows(_p(resid), _p(copy), dtype_code(copy.dtype), ctypes.c_longlong(copy.numel()), _stream()))


ACT_KINDS = {"relu2": 0, "gelu_tanh": 1, "silu": 2}


def act(x: torch.Tensor, out: torch.Tensor, kind: str) -> None:
    """out = activation(x), element by element: relu2 (the square of relu), gelu_tanh, silu."""
    _cuda(x, out)
    if x.dtype != out.dtype or x.numel() != out.numel() or kind not in ACT_KINDS:
        raise KernelError(f"act: in and out of one dtype and size, kind one of {sorted(ACT_KINDS)}")
    _check(lib().gg_act(_p(x), _p(out), dtype_code(x.dtype), ctypes.c_longlong(x.numel()), ACT_KINDS[kind], _stream()))


# ---------------------------------------------------------------- latent attention
def latent_norm_write(src: torch.Tensor, col0: int, rank: int, weight: torch.Tensor, eps: float,
                      slot_mapping: torch.Tensor, cache: torch.Tensor) -> None:
    """c[t] = rmsnorm(src[t, col0 : col0 + rank]) * weight, written to the paged cache
    [pages, 1, page, rank_padded] at slot_mapping[t] (padding columns zero; slot < 0: no write)."""
    _cuda(src, weight, slot_mapping, cache)
    if weight.dtype != torch.float32 or weight.numel() != rank or cache.dtype != src.dtype:
        raise KernelError("latent_norm_write: weight float32 [rank], cache of the source's dtype")
    _check(lib().gg_latent_norm_write(_p(src), ctypes.c_longlong(src.stride(0)), col0, rank, cache.shape[-1],
                                      _p(weight), ctypes.c_float(eps), _p(slot_mapping), _p(cache),
                                      dtype_code(src.dtype), src.shape[0], _stream()))


def grouped_gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, n: int, k: int, groups: int, *,
                 a_group_cols: int = 0, o_group_cols: int = 0, n_padded: Optional[int] = None,
                 offsets: Optional[torch.Tensor] = None, row_index: Optional[torch.Tensor] = None, row_div: int = 1,
                 rows: Optional[int] = None, gated: bool = False, gate: Optional[torch.Tensor] = None,
                 gate_col0: int = 0) -> None:
    """out_g = a_g @ w_g^T for every group g (csrc/grouped_gemm.cu).  w [groups, n (2n if gated), k].
    Without ``offsets`` every group has the first ``rows`` rows of a and reads columns
    g * a_group_cols .. + k of them; with ``offsets`` [groups + 1] group g has rows offsets[g] ..
    offsets[g + 1] of the row list (``rows`` = its length), row r reading row row_index[r] // row_div
    of a.  Results go to out[r, g * o_group_cols : + n_padded] (zeros past n).  ``gate``: row r of
    group g is multiplied by sigmoid(gate[a row, gate_col0 + g])."""
    _cuda(w, offsets, row_index)
    if a.dtype != w.dtype or out.dtype != a.dtype or a.stride(-1) != 1 or out.stride(-1) != 1:
        raise KernelError("grouped_gemm: a, w and out of one dtype, rows contiguous")
    if w.numel() != groups * (2 if gated else 1) * n * k:
        raise KernelError("grouped_gemm: w does not hold groups x n x k values")
    M = int(rows if rows is not None else a.shape[0])
    _check(lib().gg_grouped_gemm(_p(a), ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(a_group_cols), _p(row_index),
                                 int(row_div), _p(w), _p(out), ctypes.c_longlong(out.stride(0)),
                                 ctypes.c_longlong(o_group_cols), _p(offsets), M, groups, n, k,
                                 int(n_padded if n_padded is not None else n), int(gated), _p(gate),
                                 ctypes.c_longlong(gate.stride(0) if gate is not None else 0), int(gate_col0),
                                 dtype_code(a.dtype), _stream()))


def head_gate(a: torch.Tensor, gates: torch.Tensor, col0: int, heads: int) -> None:
    """a[t, h * n : h * n + n] *= sigmoid(gates[t, col0 + h]) in place (a [T, heads * n] contiguous)."""
    _cuda(a)
    T, w = a.shape
    if w % heads or gates.dtype != a.dtype or gates.stride(-1) != 1:
        raise KernelError("head_gate: a is [T, heads * n], the gates of its dtype")
    _check(lib().gg_head_gate(_p(a), _p(gates), ctypes.c_longlong(gates.stride(0)), int(col0), T, heads, w // heads,
                              dtype_code(a.dtype), _stream()))


# ---------------------------------------------------------------- mixture of experts
MOE_MAX_EXPERTS, MOE_MAX_TOP = 1024, 32


MOE_WEIGH = {"softmax_chosen": 0, "softmax_all": 1}


def moe_route(h: torch.Tensor, w_router: torch.Tensor, bias: Optional[torch.Tensor], top: int,
              idx: torch.Tensor, wgt: torch.Tensor, weigh: str = "softmax_chosen", groups: int = 1, keep: int = 1) -> None:
    """Float32 logits h @ w_router^T + bias; idx [T, top] int32 = the largest, wgt [T, top]
    float32 = softmax over those ("softmax_chosen"), or the softmax over all experts divided by the
    chosen ones' sum ("softmax_all").  ``groups`` > 1: only experts of the ``keep`` groups (of
    neighbouring experts) with the best expert can be chosen."""
    _cuda(h, w_router, bias, idx, wgt)
    T, D = h.shape
    E = w_router.shape[0]
    if w_router.dtype != h.dtype or w_router.shape[1] != D or idx.dtype != torch.int32 or wgt.dtype != torch.float32 \
            or (bias is not None and bias.dtype != torch.float32):
        raise KernelError("moe_route: router of the rows' dtype, bias and weights float32, choices int32")
    _check(lib().gg_moe_route(_p(h), _p(w_router), _p(bias), T, D, E, top, MOE_WEIGH[weigh], int(groups), int(keep),
                               _p(idx), _p(wgt), dtype_code(h.dtype), _stream()))


def moe_topk(z: torch.Tensor, bias: Optional[torch.Tensor], top: int, idx: torch.Tensor, wgt: torch.Tensor,
             weigh: str = "softmax_chosen", groups: int = 1, keep: int = 1) -> None:
    """moe_route's choice from logits z [T, E] (float32) that a product has already made."""
    _cuda(z, bias, idx, wgt)
    if z.dtype != torch.float32 or idx.dtype != torch.int32 or wgt.dtype != torch.float32:
        raise KernelError("moe_topk: logits and weights float32, choices int32")
    _check(lib().gg_moe_topk(_p(z), _p(bias), z.shape[0], z.shape[1], top, MOE_WEIGH[weigh], int(groups), int(keep),
                              _p(idx), _p(wgt), _stream()))


def moe_align(idx: torch.Tensor, n: int, experts: int, offsets: torch.Tensor, order: torch.Tensor,
              place: torch.Tensor, pad: int = 1, tile_group: Optional[torch.Tensor] = None) -> None:
    """The n (token, choice) pairs of idx sorted by expert: offsets [experts + 1], order (pair
    index at each place), place [n] (place of each pair).  ``pad`` > 1: every expert's places start
    at a multiple of pad; order then has n + experts * (pad - 1) entries or more, -1 at places
    that hold no pair, and tile_group[i] is the expert of places pad * i .. (or -1)."""
    _cuda(idx, offsets, order, place, tile_group)
    _check(lib().gg_moe_align(_p(idx), n, experts, int(pad), order.numel(), _p(offsets), _p(order), _p(place),
                              _p(tile_group), tile_group.numel() if tile_group is not None else 0, _stream()))


def moe_gather(x: torch.Tensor, order: torch.Tensor, top: int, out: torch.Tensor) -> None:
    """out[p] = x[order[p] // top] where order[p] >= 0, zeros elsewhere."""
    _cuda(x, order, out)
    if out.dtype != x.dtype or out.shape[1] != x.shape[1] or out.shape[0] != order.numel():
        raise KernelError("moe_gather: one row of x's width and dtype per place")
    _check(lib().gg_moe_gather(_p(x), _p(order), order.numel(), int(top), x.shape[1], _p(out), dtype_code(x.dtype), _stream()))


def gemm_tc_grouped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_group: torch.Tensor, groups: int,
                    gated: bool = False) -> None:
    """The tcgen05 product (gemm_tc) over groups: rows 128 i .. of x belong to group tile_group[i]
    (< 0: to none, skipped) and are multiplied with that group's matrix w[g] ([groups, N, K]; gated:
    [groups, 2N, K], out = silu(x Wg^T) * (x Wu^T)).  bfloat16; rows of x a multiple of 128."""
    global tc_launched
    M, K = x.shape
    N = out.shape[1]
    if w.numel() != groups * (2 if gated else 1) * N * K or out.shape[0] != M or not out.is_contiguous() \
            or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("gemm_tc_grouped: shapes or dtypes do not fit")
    _cuda(w, out, tile_group)
    tc_launched = True
    _check(lib().gg_gemm_tc_grouped(_p(x), ctypes.c_longlong(x.stride(0)), _p(w), _p(out), M, N, K, 2 if gated else 0,
                                    _p(tile_group), groups, _p(tc_status(x.device)), _stream()))


def moe_combine(y: torch.Tensor, place: torch.Tensor, wgt: torch.Tensor, shared: Optional[torch.Tensor],
                out: torch.Tensor, top: int) -> None:
    """out[t] = sum_j wgt[t, j] * y[place[t * top + j]] (+ shared[t])."""
    _cuda(y, place, wgt, shared, out)
    T, D = out.shape
    _check(lib().gg_moe_combine(_p(y), _p(place), _p(wgt), _p(shared), _p(out), T, D, top, dtype_code(out.dtype), _stream()))


# ---------------------------------------------------------------- attention of any make (general kernels)
def rope_kv_write_x(qkv: torch.Tensor, positions: torch.Tensor, slot_mapping: Optional[torch.Tensor],
                    inv_freq: Optional[torch.Tensor], magnitude: float, bias: Optional[torch.Tensor],
                    kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor], nh: int, nkv: int, d: int,
                    nv: int, dv: int, page_size: int, interleaved: bool = False, write_cache: bool = True) -> None:
    """Rows [nh*d | nkv*d | nv*dv] of qkv: ``bias`` (float32, the row's width) is added, the first
    2 * len(inv_freq) values of every q and k head are rotated (cosines and sines times
    ``magnitude``), k goes to kcache [pages, nkv, page, d] and v to vcache [pages, nv, page, dv]
    at slot_mapping[t]."""
    _cuda(positions, slot_mapping, inv_freq, bias, kcache, vcache)
    width = (nh + nkv) * d + nv * dv
    if qkv.stride(1) != 1 or qkv.shape[1] < width:
        raise KernelError("rope_kv_write_x: rows are not contiguous or too short")
    if inv_freq is not None and inv_freq.dtype != torch.float64:
        raise KernelError("rope_kv_write_x: inverse frequencies must be float64")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != width):
        raise KernelError("rope_kv_write_x: the bias is float32 of the row's width")
    if kcache is not None and (kcache.dtype != qkv.dtype or vcache.dtype != qkv.dtype):
        raise KernelError("rope_kv_write_x: cache and activations differ in dtype")
    rot = 2 * inv_freq.numel() if inv_freq is not None else 0
    _check(lib().gg_rope_kv_write_x(_p(qkv), ctypes.c_longlong(qkv.stride(0)), dtype_code(qkv.dtype), _p(positions),
                                    _p(slot_mapping), _p(inv_freq), ctypes.c_float(magnitude), _p(bias), _p(kcache),
                                    _p(vcache), qkv.shape[0], nh, nkv, d, nv, dv, rot, page_size, int(interleaved),
                                    int(write_cache), _stream()))


# distances whose bias the mma.sync kernels with sigmoid weights can tabulate in shared memory (attention_common.cuh)
ATTN_MMA_X_MAX_DIST = 16384


def attn_prefill_x(q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                   block_tables: torch.Tensor, bt_stride: int, cu_q_lens: torch.Tensor, context_lens: torch.Tensor,
                   tile_seq: torch.Tensor, tile_q0: torch.Tensor, num_tiles: int, out: torch.Tensor, nh: int, nkv: int,
                   d: int, dv: int, v_share: int, page_size: int, window: int, scale: float, softcap: float,
                   tile64_seq: Optional[torch.Tensor] = None, tile64_q0: Optional[torch.Tensor] = None,
                   num_tiles64: int = 0, allow_mma: bool = True, keep_first: int = 0, sigmoid_weights: bool = False,
                   head_bias: Optional[torch.Tensor] = None, dist_bias: Optional[torch.Tensor] = None,
                   dist_bucket: Optional[torch.Tensor] = None, chunk: int = 0,
                   sink: Optional[torch.Tensor] = None) -> None:
    """Causal attention of prompt portions with keys of size d, values of size dv, ``v_share`` key
    heads to a value head, optional window and capped scores; out [T, nh*dv] in the cache's type or
    float32.  ``tile_*`` list tiles of 16 queries (general kernel, float32 arithmetic), ``tile64_*``
    of 64 (mma.sync kernel: bfloat16, d and dv 64 or 128).  ``keep_first`` keys at
    the start of the sequence stay visible behind the window; ``dist_bias`` [rows, nh] float32 adds
    row dist_bucket[min(i - j, len(dist_bucket) - 1)] to the scaled score of query i and key j;
    ``sigmoid_weights``: a visible key weighs sigmoid(score + head_bias[h]) and nothing is normalised.
    With softmax these three are the general kernel's alone; with sigmoid weights the mma.sync kernel
    has them too while dist_bucket has fewer than ATTN_MMA_X_MAX_DIST entries.  ``chunk`` > 0: a query sees
    only the keys of its own chunk of that many positions (chunks counted from position 0 of the
    sequence); ``sink`` [nh] float32: exp(sink[h]) is added to the softmax denominator of head h."""
    _attn_extras(nh, head_bias, dist_bias, dist_bucket, sink)
    _check(lib().gg_attn_prefill_x(_p(q), ctypes.c_longlong(q_stride), _p(kcache), _p(vcache), dtype_code(kcache.dtype),
                                   _p(block_tables), bt_stride, _p(cu_q_lens), _p(context_lens), _p(tile_seq),
                                   _p(tile_q0), num_tiles, _p(tile64_seq), _p(tile64_q0), num_tiles64, int(allow_mma),
                                   _p(out), int(out.dtype == torch.float32 and kcache.dtype != torch.float32),
                                   nh, nkv, d, dv, v_share, page_size, window, ctypes.c_float(scale),
                                   ctypes.c_float(softcap), int(keep_first), int(sigmoid_weights), _p(head_bias),
                                   _p(dist_bias), _p(dist_bucket),
                                   dist_bucket.numel() - 1 if dist_bucket is not None else 0, int(chunk or 0), _p(sink),
                                   _stream()))


def attn_mma_x_chunk_sink() -> bool:
    """Whether the mma.sync kernels behind attn_prefill_x / attn_decode_x take ``chunk`` and ``sink``."""
    return bool(lib().gg_attn_mma_x_chunk_sink())


def _attn_extras(nh, head_bias, dist_bias, dist_bucket, sink=None) -> None:
    _cuda(head_bias, dist_bias, dist_bucket, sink)
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != nh):
        raise KernelError("attention: the sink is float32 [heads]")
    if head_bias is not None and (head_bias.dtype != torch.float32 or head_bias.numel() != nh):
        raise KernelError("attention: the bias per head is float32 [heads]")
    if dist_bias is not None and (dist_bias.dtype != torch.float32 or dist_bias.dim() != 2 or dist_bias.shape[1] != nh
                                  or dist_bucket is None or dist_bucket.dtype != torch.int32 or dist_bucket.numel() < 1):
        raise KernelError("attention: the distance bias is float32 [rows, heads] with an int32 bucket table")


def attn_decode_x(q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                  block_tables: torch.Tensor, bt_stride: int, cu_q_lens: torch.Tensor, context_lens: torch.Tensor,
                  dec_seqs: torch.Tensor, n_dec: int, num_splits: int, part_o: torch.Tensor, part_ml: torch.Tensor,
                  out: torch.Tensor, nh: int, nkv: int, d: int, dv: int, v_share: int, page_size: int, window: int,
                  scale: float, softcap: float, allow_mma: bool = True, keep_first: int = 0,
                  sigmoid_weights: bool = False, head_bias: Optional[torch.Tensor] = None,
                  dist_bias: Optional[torch.Tensor] = None, dist_bucket: Optional[torch.Tensor] = None,
                  chunk: int = 0, sink: Optional[torch.Tensor] = None) -> None:
    """The same for single decoded tokens, split over the context and merged."""
    _attn_extras(nh, head_bias, dist_bias, dist_bucket, sink)
    if part_o.numel() < n_dec * nh * num_splits * dv or part_ml.numel() < n_dec * nh * num_splits * 2:
        raise KernelError("attn_decode_x: scratch too small")
    _check(lib().gg_attn_decode_x(_p(q), ctypes.c_longlong(q_stride), _p(kcache), _p(vcache), dtype_code(kcache.dtype),
                                  _p(block_tables), bt_stride, _p(cu_q_lens), _p(context_lens), _p(dec_seqs), n_dec,
                                  num_splits, _p(part_o), _p(part_ml), _p(out),
                                  int(out.dtype == torch.float32 and kcache.dtype != torch.float32), nh, nkv, d, dv,
                                  v_share, page_size, window, ctypes.c_float(scale), ctypes.c_float(softcap),
                                  int(allow_mma), int(keep_first), int(sigmoid_weights), _p(head_bias), _p(dist_bias),
                                  _p(dist_bucket), dist_bucket.numel() - 1 if dist_bucket is not None else 0,
                                  int(chunk or 0), _p(sink), _stream()), 2)


def diff_combine(maps: torch.Tensor, out: torch.Tensor, lam: float, eps: float, post: float, heads: int,
                 kv_heads: int, dv: int) -> None:
    """maps float32 [T, 2*heads*dv] laid out [kv group][map][head in group][dv]; out[t, h] =
    rms-normed (map 1 - lam * map 2) * post, [T, heads*dv]."""
    _cuda(maps, out)
    T = out.shape[0]
    if maps.dtype != torch.float32 or maps.numel() != 2 * out.numel() or out.shape[1] != heads * dv:
        raise KernelError("diff_combine: maps float32 [T, 2 H dv], out [T, H dv]")
    _check(lib().gg_diff_combine(_p(maps), _p(out), ctypes.c_float(lam), ctypes.c_float(eps), ctypes.c_float(post),
                                 T, heads, kv_heads, dv, dtype_code(out.dtype), _stream()))


# ---------------------------------------------------------------- joining branches
def rms_mix(ys, weights, coef: float, eps: float, out: torch.Tensor) -> None:
    """out = coef * sum_i rmsnorm(ys[i]) * weights[i]; ys of out's shape and dtype, weights float32."""
    _cuda(out, *ys, *weights)
    T, W = out.shape
    n = len(ys)
    if n != len(weights) or any(y.shape != out.shape or y.dtype != out.dtype for y in ys) \
            or any(w.dtype != torch.float32 or w.numel() != W for w in weights):
        raise KernelError("rms_mix: branches of the output's shape and dtype, float32 weights of its width")
    yp = (ctypes.c_void_p * n)(*[y.data_ptr() for y in ys])
    wp = (ctypes.c_void_p * n)(*[w.data_ptr() for w in weights])
    _check(lib().gg_rms_mix(yp, wp, n, ctypes.c_float(coef), ctypes.c_float(eps), T, W, dtype_code(out.dtype),
                            _p(out), _stream()))


def scaled_add(resid: torch.Tensor, a: torch.Tensor, b: Optional[torch.Tensor], mult: float,
               bias: Optional[torch.Tensor] = None) -> None:
    """resid += mult * (a + b + bias): resid float32 [T, W], a and b of one dtype, bias float32 [W]."""
    _cuda(resid, a, b, bias)
    T, W = resid.shape
    if resid.dtype != torch.float32 or a.shape != resid.shape or (b is not None and (b.shape != a.shape or b.dtype != a.dtype)):
        raise KernelError("scaled_add: float32 residual, sublayer outputs of its shape and one dtype")
    _check(lib().gg_scaled_add(_p(resid), _p(a), _p(b), _p(bias), ctypes.c_float(mult), T, W, dtype_code(a.dtype), _stream()))


def bias_add(y: torch.Tensor, bias: torch.Tensor) -> None:
    """y[t, :] += bias (float32 [W]), in place."""
    _cuda(y, bias)
    if bias.dtype != torch.float32 or bias.numel() != y.shape[1]:
        raise KernelError("bias_add: float32 bias of the rows' width")
    _check(lib().gg_bias_add(_p(y), _p(bias), y.shape[0], y.shape[1], dtype_code(y.dtype), _stream()))


def concat_cast(a: torch.Tensor, delta: Optional[torch.Tensor], b: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = [a[t] (+ delta[t]), b[t]] rounded to out's dtype; a, b float32 [T, W], out [T, 2W]."""
    _cuda(a, delta, b, out)
    T, W = a.shape
    if a.dtype != torch.float32 or b.dtype != torch.float32 or b.shape != a.shape or out.shape != (T, 2 * W) \
            or (delta is not None and (delta.dtype != out.dtype or delta.shape != a.shape)):
        raise KernelError("concat_cast: two float32 [T, W] in, [T, 2W] out")
    _check(lib().gg_concat_cast(_p(a), _p(delta), _p(b), _p(out), T, W, dtype_code(out.dtype), _stream()))


def clamped_gate(gate_up: torch.Tensor, out: torch.Tensor, limit: float, alpha: float, shift: float) -> None:
    """g = min(gate, limit), u = clamp(up, -limit, limit): out = g * sigmoid(alpha * g) * (u + shift);
    gate_up [T, 2I] (gates, then ups), out [T, I]."""
    _cuda(gate_up, out)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I) or gate_up.dtype != out.dtype:
        raise KernelError("clamped_gate: input must be [T, 2I] of the output's dtype")
    _check(lib().gg_clamped_gate(_p(gate_up), _p(out), T, I, ctypes.c_float(limit), ctypes.c_float(alpha),
                                 ctypes.c_float(shift), dtype_code(out.dtype), _stream()))


# ---------------------------------------------------------------- gated delta rule
def delta_prep(x: torch.Tensor, conv_w: torch.Tensor, conv_state: torch.Tensor, zb: torch.Tensor, za: torch.Tensor,
               a_log: torch.Tensor, dt_bias: torch.Tensor, cu_q_lens: torch.Tensor, context_lens: torch.Tensor,
               state_slots: torch.Tensor, num_seqs: int, kv_heads: int, heads: int, d: int, dv: int,
               qkv_out: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor) -> None:
    """Short convolution + SiLU of the q, k, v channels of x [T, >= C] (C = 2*kv_heads*d + heads*dv)
    with the window carried in conv_state [slots, taps-1, C]; q and k made unit vectors (q times
    d^-1/2); beta = sigmoid(zb) [T, H], decay = exp(-exp(a_log) * softplus(za + dt_bias)) where za and
    decay are [T, H] (a decay per head) or [T, H * d] (per head and key channel; dt_bias then [H * d]).
    zb and za may be column views of one float32 buffer.  Then the window is moved on.  Outputs float32."""
    _cuda(conv_w, conv_state, a_log, dt_bias, qkv_out, beta, decay)
    C, taps = conv_w.shape
    if x.stride(1) != 1 or C != 2 * kv_heads * d + heads * dv or conv_w.dtype != torch.float32 \
            or conv_state.dtype != torch.float32 or zb.dtype != torch.float32 or za.dtype != torch.float32 \
            or qkv_out.dtype != torch.float32 or zb.stride(1) != 1 or za.stride(1) != 1 or zb.shape[1] != heads:
        raise KernelError("delta_prep: bad shapes or dtypes")
    dw = za.shape[1] // heads
    if za.shape[1] != heads * dw or dt_bias.numel() != heads * dw or decay.numel() != x.shape[0] * heads * dw:
        raise KernelError("delta_prep: the decay's input, bias and output disagree in width")
    _check(lib().gg_delta_prep(_p(x), ctypes.c_longlong(x.stride(0)), dtype_code(x.dtype), _p(conv_w), _p(conv_state),
                               _p(zb), ctypes.c_longlong(zb.stride(0)), _p(za), ctypes.c_longlong(za.stride(0)), dw,
                               _p(a_log), _p(dt_bias), _p(cu_q_lens), _p(context_lens), _p(state_slots),
                               x.shape[0], num_seqs, kv_heads, heads, d, dv, taps, _p(qkv_out), _p(beta), _p(decay),
                               _stream()), 2 if taps > 1 else 1)


def delta_recur(qkv: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
                cu_q_lens: torch.Tensor, context_lens: torch.Tensor, state_slots: torch.Tensor, num_seqs: int,
                kv_heads: int, heads: int, d: int, dv: int, o_raw: torch.Tensor, plain: bool = False) -> None:
    """The recurrence S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q over every sequence's
    tokens of the step, from and to state [slots, heads, dv, d] float32.  decay [T, heads]: g is a
    number per head; [T, heads * d]: a factor per key channel (row of S).  ``plain``: u = beta v (the
    write does not look at the state: the recurrence of a state-space layer)."""
    _cuda(qkv, beta, decay, state, o_raw)
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (heads, dv, d):
        raise KernelError("delta_recur: state must be float32 [slots, heads, dv, d]")
    dw = decay.shape[-1] // heads
    _check(lib().gg_delta_recur(_p(qkv), _p(beta), _p(decay), _p(state), _p(cu_q_lens), _p(context_lens),
                                _p(state_slots), num_seqs, kv_heads, heads, d, dv, dw, int(plain), o_raw.shape[0], _p(o_raw),
                                _stream()))


def delta_out(o_raw: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, heads: int, dv: int,
              out: torch.Tensor, gate_act: str = "silu") -> None:
    """out[t, h] = o / sqrt(mean(o^2) + eps) * weight * act(gate[t, h]), act = silu or sigmoid; gate is
    a column view [T, heads*dv] of a projection's output."""
    _cuda(o_raw, weight, out)
    if gate.stride(1) != 1 or gate.dtype != out.dtype or weight.dtype != torch.float32:
        raise KernelError("delta_out: gate rows contiguous and of the output's dtype, float32 weight")
    _check(lib().gg_delta_out(_p(o_raw), _p(gate), ctypes.c_longlong(gate.stride(0)), dtype_code(out.dtype), _p(weight),
                              ctypes.c_float(eps), out.shape[0], heads, dv, {"silu": 0, "sigmoid": 1}[gate_act],
                              _p(out), _stream()))


# ---------------------------------------------------------------- state-space layer
def ssm_prep(proj: torch.Tensor, conv_w: torch.Tensor, conv_b: Optional[torch.Tensor], conv_state: Optional[torch.Tensor],
             a_log: torch.Tensor, dt_bias: torch.Tensor, cu_q_lens: torch.Tensor, context_lens: torch.Tensor,
             state_slots: torch.Tensor, num_seqs: int, heads: int, vdim: int, groups: int, state: int,
             cbx: torch.Tensor, dt: torch.Tensor, decay: torch.Tensor) -> None:
    """Rows [z | x | B | C | dt] of proj: short convolution (+ bias) and SiLU over the x, B, C channels
    with the window carried in conv_state [slots, taps-1, channels]; cbx [T, channels] float32 gets them
    in the order [C | B | x]; dt = softplus(dt + dt_bias), decay = exp(-exp(a_log) dt), both [T, heads]
    float32.  Then the window is moved on."""
    _cuda(conv_w, conv_b, conv_state, a_log, dt_bias, cbx, dt, decay)
    Cc, taps = conv_w.shape
    if proj.stride(1) != 1 or Cc != heads * vdim + 2 * groups * state or conv_w.dtype != torch.float32 \
            or cbx.dtype != torch.float32 or dt.dtype != torch.float32 or decay.dtype != torch.float32 \
            or (conv_state is not None and conv_state.dtype != torch.float32):
        raise KernelError("ssm_prep: bad shapes or dtypes")
    _check(lib().gg_ssm_prep(_p(proj), ctypes.c_longlong(proj.stride(0)), dtype_code(proj.dtype), _p(conv_w), _p(conv_b),
                             _p(conv_state), _p(a_log), _p(dt_bias), _p(cu_q_lens), _p(context_lens), _p(state_slots),
                             proj.shape[0], num_seqs, heads, vdim, groups, state, taps, _p(cbx), _p(dt), _p(decay),
                             _stream()), 2 if taps > 1 else 1)


def ssm_out(y_raw: torch.Tensor, cbx: torch.Tensor, x_col: int, z: torch.Tensor, D: torch.Tensor, weight: torch.Tensor,
            eps: float, heads: int, vdim: int, parts: int, out: torch.Tensor) -> None:
    """out = rms-normed in ``parts`` equal parts of ((y_raw + D[h] x) * silu(z)), times weight; x is
    cbx[:, x_col:], z a column view [T, heads*vdim] of the projection's output."""
    _cuda(y_raw, cbx, D, weight, out)
    if z.stride(1) != 1 or z.dtype != out.dtype or weight.dtype != torch.float32 or D.dtype != torch.float32:
        raise KernelError("ssm_out: gate rows contiguous and of the output's dtype, float32 weight and D")
    _check(lib().gg_ssm_out(_p(y_raw), _p(cbx), int(x_col), cbx.shape[1], _p(z), ctypes.c_longlong(z.stride(0)),
                            dtype_code(out.dtype), _p(D), _p(weight), ctypes.c_float(eps), out.shape[0], heads, vdim,
                            int(parts), _p(out), _stream()))


# ---------------------------------------------------------------- more small row kernels
def weighted_sum(ys, coefs, out: torch.Tensor) -> None:
    """out = sum_i coefs[i] * ys[i]; ys of out's shape and dtype."""
    _cuda(out, *ys)
    n = len(ys)
    if n != len(coefs) or any(y.shape != out.shape or y.dtype != out.dtype for y in ys):
        raise KernelError("weighted_sum: branches of the output's shape and dtype, a factor each")
    yp = (ctypes.c_void_p * n)(*[y.data_ptr() for y in ys])
    cf = (ctypes.c_float * n)(*[float(c) for c in coefs])
    _check(lib().gg_weighted_sum(yp, cf, n, out.shape[0], out.shape[1], dtype_code(out.dtype), _p(out), _stream()))


def token_shift(h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, cu_q_lens: torch.Tensor,
                context_lens: torch.Tensor, state_slots: torch.Tensor, num_seqs: int, out: torch.Tensor) -> None:
    """out[t] = h[t] + (h[t-1] - h[t]) * mu; the row before a portion's first comes from
    state[slot] (float32 [slots, W]; zeros at the start of a sequence), which then takes the portion's last row."""
    _cuda(h, mu, state, out)
    T, W = h.shape
    if out.shape != h.shape or out.dtype != h.dtype or mu.dtype != torch.float32 or mu.numel() != W \
            or state.dtype != torch.float32 or state.shape[-1] != W:
        raise KernelError("token_shift: rows and result of one shape and dtype, float32 factors and state of their width")
    _check(lib().gg_token_shift(_p(h), _p(mu), _p(state), _p(cu_q_lens), _p(context_lens), _p(state_slots), T, num_seqs,
                                W, dtype_code(h.dtype), _p(out), _stream()))


def softcap(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap) in place (float32)."""
    _cuda(x)
    if x.dtype != torch.float32:
        raise KernelError("softcap: float32 values")
    _check(lib().gg_softcap(_p(x), ctypes.c_longlong(x.numel()), ctypes.c_float(cap), _stream()))


def scale_add_rows(resid: torch.Tensor, scale: float, table: torch.Tensor, positions: torch.Tensor,
                   bad: Optional[torch.Tensor] = None) -> None:
    """resid[t] = resid[t] * scale + table[positions[t]] (resid float32 [T, W], table [rows, W])."""
    _cuda(resid, table, positions, bad)
    T, W = resid.shape
    if resid.dtype != torch.float32 or table.shape[1] != W or positions.dtype != torch.int32:
        raise KernelError("scale_add_rows: float32 rows, a table of their width, int32 positions")
    _check(lib().gg_scale_add_rows(_p(resid), ctypes.c_float(scale), _p(table), _p(positions), T, W, table.shape[0],
                                   dtype_code(table.dtype), _p(bad), _stream()))


def sigmoid_gate(a: torch.Tensor, gate: torch.Tensor, out: torch.Tensor) -> None:
    """out = a * sigmoid(gate): a float32 [T, W], gate a column view [T, W] of the activation type, out of that type."""
    _cuda(a, out)
    if a.dtype != torch.float32 or gate.dtype != out.dtype or gate.stride(1) != 1 or gate.shape != a.shape or out.shape != a.shape:
        raise KernelError("sigmoid_gate: float32 values, gate and result of the activation type and one shape")
    _check(lib().gg_sigmoid_gate(_p(a), _p(gate), ctypes.c_longlong(gate.stride(0)), _p(out), a.shape[0], a.shape[1],
                                 dtype_code(out.dtype), _stream()))


# ---------------------------------------------------------------- normed heads, rotated latent parts, gates
def qkv_norm_rope_write(qkv: torch.Tensor, positions: torch.Tensor, slot_mapping: Optional[torch.Tensor],
                        inv_freq: Optional[torch.Tensor], magnitude: float, q_weight: Optional[torch.Tensor],
                        k_weight: Optional[torch.Tensor], eps: float, v_unit: bool, v_first: Optional[torch.Tensor],
                        mix: int, lam: float, kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor], nh: int,
                        nkv: int, d: int, nv: int, dv: int, page_size: int, interleaved: bool = False,
                        write_cache: bool = True) -> None:
    """Rows [nh*d | nkv*d | nv*dv] of qkv: every q and k head divided by its root mean square and
    multiplied by q_weight / k_weight (float32 [d]; None: no norm), then rotated (the first
    2 * len(inv_freq) values; cosines and sines times ``magnitude``): q in place, k to kcache.  Every v
    head divided by its root mean square if ``v_unit``; ``mix`` 1: the result is also stored in v_first
    (float32 [T, nv*dv]); 2: it is blended (1 - lam) v + lam v_first; then v goes to vcache."""
    _cuda(positions, slot_mapping, inv_freq, q_weight, k_weight, v_first, kcache, vcache)
    width = (nh + nkv) * d + nv * dv
    if qkv.stride(1) != 1 or qkv.shape[1] < width:
        raise KernelError("qkv_norm_rope_write: rows are not contiguous or too short")
    if inv_freq is not None and inv_freq.dtype != torch.float64:
        raise KernelError("qkv_norm_rope_write: inverse frequencies must be float64")
    for w in (q_weight, k_weight):
        if w is not None and (w.dtype != torch.float32 or w.numel() != d):
            raise KernelError("qkv_norm_rope_write: a norm weight is float32 [head size]")
    if v_first is not None and (v_first.dtype != torch.float32 or v_first.numel() < qkv.shape[0] * nv * dv):
        raise KernelError("qkv_norm_rope_write: the first layer's values are float32 [T, nv * dv]")
    if kcache is not None and (kcache.dtype != qkv.dtype or vcache.dtype != qkv.dtype):
        raise KernelError("qkv_norm_rope_write: cache and activations differ in dtype")
    rot = 2 * inv_freq.numel() if inv_freq is not None else 0
    _check(lib().gg_qkv_norm_rope_write(_p(qkv), ctypes.c_longlong(qkv.stride(0)), dtype_code(qkv.dtype), _p(positions),
                                        _p(slot_mapping), _p(inv_freq), ctypes.c_float(magnitude), _p(q_weight),
                                        _p(k_weight), ctypes.c_float(eps), int(v_unit), int(mix), ctypes.c_float(lam),
                                        _p(v_first), _p(kcache), _p(vcache), qkv.shape[0], nh, nkv, d, nv, dv, rot,
                                        page_size, int(interleaved), int(write_cache), _stream()))


def latent_rope(src: torch.Tensor, k_col0: int, q_head: int, q_off: int, heads: int, positions: torch.Tensor,
                inv_freq: torch.Tensor, magnitude: float, interleaved: bool, slot_mapping: Optional[torch.Tensor],
                cache: Optional[torch.Tensor], qout: torch.Tensor, row: int, dst_col: int, write_cache: bool = True) -> None:
    """The rotated parts of a latent attention: columns [k_col0, + rot) of src[t] (the key part all heads share) go,
    rotated, to columns [dst_col, + rot) of the cache row (``row`` values) at slot_mapping[t]; columns
    [h * q_head + q_off, + rot) (head h's query part) to columns [h * row + dst_col, + rot) of qout[t]."""
    _cuda(positions, inv_freq, slot_mapping, cache)
    rot = 2 * inv_freq.numel()
    if src.stride(1) != 1 or qout.stride(1) != 1 or qout.dtype != src.dtype or inv_freq.dtype != torch.float64 \
            or (cache is not None and (cache.dtype != src.dtype or cache.shape[-1] != row)):
        raise KernelError("latent_rope: rows contiguous and of one dtype, float64 frequencies, cache rows of the given width")
    _check(lib().gg_latent_rope(_p(src), ctypes.c_longlong(src.stride(0)), int(k_col0), int(q_head), int(q_off), heads, rot,
                                _p(positions), _p(inv_freq), ctypes.c_float(magnitude), int(interleaved), _p(slot_mapping),
                                _p(cache), _p(qout), ctypes.c_longlong(qout.stride(0)), int(row), int(dst_col),
                                int(write_cache), dtype_code(src.dtype), src.shape[0], _stream()))


GATED_ACT_KINDS = {"relu": 0, "gelu_tanh": 1, "silu": 2}


def gated_act(gate_up: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, kind: str) -> None:
    """out[t, i] = act(gate_up[t, i] + bias[i]) * (gate_up[t, I + i] + bias[I + i]); bias float32 [2I] or None."""
    _cuda(gate_up, bias, out)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I) or gate_up.dtype != out.dtype or kind not in GATED_ACT_KINDS \
            or (bias is not None and (bias.dtype != torch.float32 or bias.numel() != 2 * I)):
        raise KernelError(f"gated_act: [T, 2I] in, [T, I] out of one dtype, float32 bias [2I], kind one of {sorted(GATED_ACT_KINDS)}")
    _check(lib().gg_gated_act(_p(gate_up), _p(bias), _p(out), T, I, GATED_ACT_KINDS[kind], dtype_code(out.dtype), _stream()),
           -(-T // 65535))


def gate_mul(a: torch.Tensor, gate: torch.Tensor) -> None:
    """a *= sigmoid(gate) in place: a [T, W] contiguous, gate a column view [T, W] of the same dtype."""
    _cuda(a)
    if gate.dtype != a.dtype or gate.stride(1) != 1 or gate.shape != a.shape:
        raise KernelError("gate_mul: values and gate of one dtype and shape")
    _check(lib().gg_gate_mul(_p(a), _p(gate), ctypes.c_longlong(gate.stride(0)), a.shape[0], a.shape[1],
                             dtype_code(a.dtype), _stream()))


def gate_norm_add(resid: torch.Tensor, y: torch.Tensor, y_bias: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                  gate_bias: Optional[torch.Tensor], weight: torch.Tensor, eps: float) -> None:
    """resid += rmsnorm((y + y_bias) * sigmoid(gate + gate_bias)) * weight: resid float32 [T, H], y and gate
    (a column view) of the activation type, the biases and the weight float32 [H]; gate None: no gate."""
    _cuda(resid, y, y_bias, gate_bias, weight)
    T, H = y.shape
    if resid.dtype != torch.float32 or resid.shape != y.shape or weight.dtype != torch.float32 or weight.numel() != H:
        raise KernelError("gate_norm_add: float32 residual of the input's shape, float32 weight of its width")
    if gate is not None and (gate.dtype != y.dtype or gate.stride(1) != 1 or gate.shape != y.shape):
        raise KernelError("gate_norm_add: the gate has the input's dtype and shape")
    for b in (y_bias, gate_bias):
        if b is not None and (b.dtype != torch.float32 or b.numel() != H):
            raise KernelError("gate_norm_add: biases are float32 of the input's width")
    _check(lib().gg_gate_norm_add(_p(resid), _p(y), _p(y_bias), _p(gate),
                                  ctypes.c_longlong(gate.stride(0) if gate is not None else 0), _p(gate_bias), _p(weight),
                                  dtype_code(y.dtype), T, H, ctypes.c_float(eps), _stream()))


# ---------------------------------------------------------------- matrix memory with exponential gates
def mlstm_gates(zi: torch.Tensor, zf: torch.Tensor, bias_i: Optional[torch.Tensor], bias_f: Optional[torch.Tensor],
                cap: float, m_state: torch.Tensor, cu_q_lens: torch.Tensor, context_lens: torch.Tensor,
                state_slots: torch.Tensor, num_seqs: int, heads: int, beta: torch.Tensor, decay: torch.Tensor,
                m_out: torch.Tensor) -> None:
    """i = cap tanh((zi + bias_i) / cap), f = logsigmoid(cap tanh((zf + bias_f) / cap)); per sequence and head
    m_t = max(f_t + m_{t-1}, i_t) from m_state [slots, heads] (0 for a new sequence), which is moved on;
    beta = exp(i - m_t), decay = exp(f + m_{t-1} - m_t), m_out = m_t, all float32 [T, heads].  zi and zf may
    be column views of one float32 buffer."""
    _cuda(bias_i, bias_f, m_state, beta, decay, m_out)
    if zi.dtype != torch.float32 or zf.dtype != torch.float32 or zi.stride(1) != 1 or zf.stride(1) != 1 \
            or m_state.dtype != torch.float32 or m_state.shape[-1] != heads:
        raise KernelError("mlstm_gates: float32 gate rows, m_state float32 [slots, heads]")
    _check(lib().gg_mlstm_gates(_p(zi), ctypes.c_longlong(zi.stride(0)), _p(zf), ctypes.c_longlong(zf.stride(0)), _p(bias_i),
                                _p(bias_f), ctypes.c_float(cap), _p(m_state), _p(cu_q_lens), _p(context_lens),
                                _p(state_slots), num_seqs, heads, beta.shape[0], _p(beta), _p(decay), _p(m_out), _stream()))


def mlstm_rows(x: torch.Tensor, heads: int, d: int, dv: int, dvp: int, qscale: float, out: torch.Tensor) -> None:
    """Rows [q | k | v] of x (heads x d, heads x d, heads x dv) to float32 rows [q * qscale | k | per head: v, 1,
    zeros up to dvp]."""
    _cuda(out)
    if x.stride(1) != 1 or out.dtype != torch.float32 or out.shape[1] != heads * (2 * d + dvp):
        raise KernelError("mlstm_rows: contiguous rows in, float32 [T, heads * (2 d + dvp)] out")
    _check(lib().gg_mlstm_rows(_p(x), ctypes.c_longlong(x.stride(0)), dtype_code(x.dtype), x.shape[0], heads, d, dv, dvp,
                               ctypes.c_float(qscale), _p(out), _stream()))


def mlstm_out(o_raw: torch.Tensor, m_row: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float,
              floor: float, heads: int, dv: int, dvp: int, out: torch.Tensor) -> None:
    """out[t, h] = unit_rms(o[:dv] / (max(|o[dv]|, exp(-m)) + floor)) * weight[h] * sigmoid(gate[t, h]); o = o_raw[t, h]
    (dvp values: column dv is the normaliser's dot product), gate a column view [T, heads*dv] of out's dtype."""
    _cuda(o_raw, m_row, weight, out)
    if gate.stride(1) != 1 or gate.dtype != out.dtype or weight.dtype != torch.float32 or weight.numel() != heads * dv:
        raise KernelError("mlstm_out: gate rows contiguous and of the output's dtype, float32 weight [heads * dv]")
    _check(lib().gg_mlstm_out(_p(o_raw), _p(m_row), _p(gate), ctypes.c_longlong(gate.stride(0)), dtype_code(out.dtype),
                              _p(weight), ctypes.c_float(eps), ctypes.c_float(floor), out.shape[0], heads, dv, dvp, _p(out),
                              _stream()))
