"""Python side of the CUDA kernels: one function per launcher in ``csrc/``.

Every function takes CUDA tensors, launches on torch's current stream and raises on
any error.  There is no CPU path and no library fallback here: a tensor that is not
on a CUDA device, or a kernel library that cannot be built or loaded, is an error.
"""
from __future__ import annotations

import ctypes
import os as _os
from typing import Optional

import torch

from .csrc.build import library, loaded as _library_loaded

F32, BF16 = 0, 1
ERR_UNSUPPORTED = 10001


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {dt}")


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise KernelError("kernel argument is not on a CUDA device (there is no CPU path)")
    return ctypes.c_void_p(t.data_ptr())


_launch_count = [0]


def launches() -> int:
    """How many kernels of this package have been launched (replays of captured steps included)."""
    return _launch_count[0]


def add_launches(n: int) -> None:
    _launch_count[0] += n


_step_stream = [None]


class step_stream:
    """Within this context every launcher uses the stream that was current on entry, looked up once:
    asking torch for the current stream costs several microseconds, a step has hundreds of launches.
    (Nothing inside a step switches streams; a graph capture enters the context after it has begun.)"""

    def __enter__(self):
        self.previous = _step_stream[0]
        _step_stream[0] = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        _step_stream[0] = self.previous
        return False


def _stream():
    _launch_count[0] += 1          # every launcher fetches the stream exactly once
    s = _step_stream[0]
    return s if s is not None else ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(code: int, what: str) -> None:
    if code == 0:
        return
    if code == ERR_UNSUPPORTED:
        raise KernelError(f"{what}: the kernel refuses these sizes or types")
    raise KernelError(f"{what}: CUDA error {code}")


def _contig(t: torch.Tensor, name: str) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


_I, _LL, _F = ctypes.c_int, ctypes.c_longlong, ctypes.c_float


# ------------------------------------------------------------------ elementwise
def embedding(x_out: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor, scale: float = 1.0) -> None:
    """x_out[t, :] = table[tokens[t], :] * scale; x_out float32 [T, D], tokens int32 [T]."""
    T, D = x_out.shape
    assert x_out.dtype == torch.float32 and tokens.dtype == torch.int32 and table.shape[1] == D
    _contig(x_out, "x_out"); _contig(table, "table")
    _check(library("elementwise").qd_embedding_scaled(_ptr(x_out), _ptr(table), _I(dtype_code(table.dtype)),
                                                      _ptr(tokens), _I(T), _I(D), _F(scale), _stream()), "embedding")


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None, write_back: bool = True,
                delta_scale: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[s] + delta[s]) * weight with s = rows[r] (or r); x float32 [T, D] is
    updated to x + delta when ``write_back``.  ``delta_scale`` (float32 [D]): delta is multiplied by it,
    element by element along D, before it is added."""
    D = x.shape[1]
    n_rows = out.shape[0]
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == D
    assert out.shape[1] == D and (rows is None or (rows.dtype == torch.int32 and rows.numel() == n_rows))
    assert rows is not None or n_rows == x.shape[0]
    _contig(x, "x"); _contig(out, "out")
    n_parts = 1
    if delta is not None:
        # delta [T, D], or float32 partial sums [n_parts, T, D] that the kernel adds up
        if delta.dim() == 3:
            n_parts = delta.shape[0]
            assert delta.dtype == torch.float32 and tuple(delta.shape[1:]) == tuple(x.shape)
        else:
            assert delta.shape == x.shape
        _contig(delta, "delta")
    if delta_scale is not None and delta is not None:
        assert delta_scale.dtype == torch.float32 and delta_scale.numel() == D and delta_scale.is_contiguous()
        _check(library("elementwise").qd_add_rmsnorm_scaled(
            _ptr(x), _ptr(delta), _I(dtype_code(delta.dtype)), _ptr(delta_scale), _ptr(weight),
            _ptr(out), _I(dtype_code(out.dtype)), _ptr(rows), _I(n_rows), _I(D), _F(eps),
            _I(1 if write_back else 0), _I(n_parts), _LL(x.numel()), _stream()), "add_rmsnorm")
        return
    _check(library("elementwise").qd_add_rmsnorm(
        _ptr(x), _ptr(delta), _I(dtype_code(delta.dtype) if delta is not None else -1), _ptr(weight),
        _ptr(out), _I(dtype_code(out.dtype)), _ptr(rows), _I(n_rows), _I(D), _F(eps),
        _I(1 if write_back else 0), _I(n_parts), _LL(x.numel()), _stream()), "add_rmsnorm")


def residual_add(x: torch.Tensor, delta: torch.Tensor, delta_scale: Optional[torch.Tensor] = None) -> None:
    """x += delta (delta [T, D], or float32 partial sums [n_parts, T, D]), times ``delta_scale`` [D] if given."""
    n_parts = delta.shape[0] if delta.dim() == 3 else 1
    assert x.dtype == torch.float32 and tuple(x.shape) == tuple(delta.shape[-2:])
    _contig(x, "x"); _contig(delta, "delta")
    if delta_scale is not None:
        assert delta_scale.dtype == torch.float32 and delta_scale.numel() == x.shape[1]
        _check(library("elementwise").qd_residual_add_scaled(
            _ptr(x), _ptr(delta), _I(dtype_code(delta.dtype)), _LL(x.numel()), _I(n_parts), _ptr(delta_scale),
            _I(x.shape[1]), _stream()), "residual_add")
        return
    _check(library("elementwise").qd_residual_add(_ptr(x), _ptr(delta), _I(dtype_code(delta.dtype)),
                                                  _LL(x.numel()), _I(n_parts), _stream()), "residual_add")


def rope_kv_write_partial(part: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor, H: int, G: int,
                          d: int, rotary_dim: int, pairing: int, cos: Optional[torch.Tensor],
                          sin: Optional[torch.Tensor], positions: torch.Tensor, kv: Optional[torch.Tensor],
                          slot_map: Optional[torch.Tensor], page_size: int, write_kv: bool) -> None:
    """As ``rope_kv_write`` from float32 partial sums part [n_parts, T, (H+2G)*d] (+ bias): rotated q goes
    to q_out bfloat16 [T, H*d], k and v to the cache."""
    n_parts, T, W = part.shape
    assert part.dtype == torch.float32 and W == (H + 2 * G) * d and q_out.shape == (T, H * d)
    assert q_out.dtype == torch.bfloat16 and positions.dtype == torch.int32
    _contig(part, "part"); _contig(q_out, "q_out")
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == W
    if write_kv:
        assert kv.dtype == torch.bfloat16 and tuple(kv.shape[1:]) == (2, G, page_size, d)
        _contig(kv, "kv")
    _check(library("elementwise").qd_rope_kv_write_partial(
        _ptr(part), _I(n_parts), _ptr(bias), _ptr(q_out), _I(T), _I(H), _I(G), _I(d), _I(rotary_dim),
        _I(pairing), _ptr(cos), _ptr(sin), _ptr(positions), _ptr(kv), _ptr(slot_map), _I(page_size),
        _I(1 if write_kv else 0), _stream()), "rope_kv_write_partial")


def rope_kv_write(qkv: torch.Tensor, H: int, G: int, d: int, rotary_dim: int, pairing: int,
                  cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor,
                  kv: Optional[torch.Tensor], slot_map: Optional[torch.Tensor], page_size: int,
                  write_kv: bool) -> None:
    """Rotate q and k of qkv [T, (H+2G)*d] in place by the table rows of ``positions`` and
    write k, v to their slots of ``kv`` [pages, 2, G, page_size, d]."""
    T = qkv.shape[0]
    assert qkv.shape[1] == (H + 2 * G) * d and positions.dtype == torch.int32
    _contig(qkv, "qkv")
    if cos is not None:
        assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.shape[1] == rotary_dim // 2
    if write_kv:
        assert kv is not None and kv.dtype == qkv.dtype and slot_map.dtype == torch.int32
        assert tuple(kv.shape[1:]) == (2, G, page_size, d), (kv.shape, G, page_size, d)
        _contig(kv, "kv")
    _check(library("elementwise").qd_rope_kv_write(
        _ptr(qkv), _I(dtype_code(qkv.dtype)), _I(T), _I(H), _I(G), _I(d), _I(rotary_dim), _I(pairing),
        _ptr(cos), _ptr(sin), _ptr(positions), _ptr(kv), _ptr(slot_map), _I(page_size),
        _I(1 if write_kv else 0), _stream()), "rope_kv_write")


def rope_kv_write_biased(qkv: torch.Tensor, bias: Optional[torch.Tensor], H: int, G: int, d: int, rotary_dim: int,
                         pairing: int, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                         positions: torch.Tensor, kv: Optional[torch.Tensor], slot_map: Optional[torch.Tensor],
                         page_size: int, write_kv: bool) -> None:
    """``rope_kv_write`` with the projection's float32 bias [(H+2G)*d] added first (rounded to bfloat16 before
    the rotation); bfloat16 and the vectorized kernel's sizes only (KernelError otherwise)."""
    T = qkv.shape[0]
    assert qkv.dtype == torch.bfloat16 and qkv.shape[1] == (H + 2 * G) * d and positions.dtype == torch.int32
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == (H + 2 * G) * d)
    _contig(qkv, "qkv")
    if write_kv:
        assert kv is not None and kv.dtype == qkv.dtype and tuple(kv.shape[1:]) == (2, G, page_size, d)
        _contig(kv, "kv")
    _check(library("elementwise").qd_rope_kv_write_biased(
        _ptr(qkv), _ptr(bias), _I(T), _I(H), _I(G), _I(d), _I(rotary_dim), _I(pairing), _ptr(cos), _ptr(sin),
        _ptr(positions), _ptr(kv), _ptr(slot_map), _I(page_size), _I(1 if write_kv else 0), _stream()),
        "rope_kv_write_biased")


def elementwise_plain_next() -> None:
    """The next launch of the elementwise library (the norm or the addition that takes a branch's output) is
    ordered after all earlier work of the stream, without programmatic dependent launch: for the reader of a
    batched library product."""
    fn = library("elementwise").qd_elementwise_plain_next
    fn.restype = None
    fn()


def swiglu_partial(part: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, f] = silu(sum_p part[p, t, f]) * (sum_p part[p, t, F + f]) from the float32 partial sums
    [n_parts, T, 2F] of a split-K gate/up product; out bfloat16."""
    T, F = out.shape
    assert part.dim() == 3 and tuple(part.shape[1:]) == (T, 2 * F) and part.dtype == torch.float32
    assert out.dtype == torch.bfloat16 and F % 4 == 0
    _contig(part, "part"); _contig(out, "out")
    _check(library("elementwise").qd_swiglu_partial(_ptr(part), _I(part.shape[0]), _ptr(out), _I(T), _I(F), _stream()),
           "swiglu_partial")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, f] = silu(gate_up[t, f]) * gate_up[t, F + f]."""
    T, F = out.shape
    assert gate_up.shape == (T, 2 * F) and gate_up.dtype == out.dtype
    _contig(gate_up, "gate_up"); _contig(out, "out")
    _check(library("elementwise").qd_swiglu(_ptr(gate_up), _ptr(out), _I(dtype_code(out.dtype)), _I(T),
                                            _I(F), _stream()), "swiglu")


# ------------------------------------------------------------------------ gemm
def gemm_generic(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[T, N] = x[T, K] @ w[N, K]^T (+ bias), float32 FMA; x and out may be row-strided."""
    T, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (T, N) and x.dtype == w.dtype
    assert x.stride(1) == 1 and out.stride(1) == 1
    _contig(w, "w")
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    _check(library("gemm_generic").qd_gemm_generic(
        _ptr(x), _ptr(w), _I(dtype_code(x.dtype)), _ptr(bias), _ptr(out), _I(dtype_code(out.dtype)),
        _I(T), _I(N), _I(K), _LL(x.stride(0)), _LL(out.stride(0)), _stream()), "gemm_generic")


SKINNY_MAX_TOKENS = 64      # what the mma.sync few-token kernels take
# Who takes a product of T tokens was settled by measurement in whole decode steps (profiles/); the numbers are
# module attributes so that a measurement can move them, not switches of the environment.
SKINNY_POLICY_TOKENS = 16      # up to here the few-token kernels are the faster choice
STREAM_POLICY_TOKENS = 8       # up to here the streaming kernel takes every product
STREAM_RESIDENT_TOKENS = 16    # from there up to here it still takes a product whose result is partial sums over
# shares of K of one stage (1,024) each: the tokens' rows for such a share stay in shared memory as whole rows do
# for up to 8 tokens (a decode step at batch 16: 2.47 -> 2.13 ms at the 3B sizes, 5.33 -> 3.56 ms at the 7B sizes);
# the other products of 9 to 16 tokens (whole sums: the output projection over the vocabulary) take the
# register-load kernel
STREAM_RESIDENT_MAX_SHARES = 32
TC5_POLICY_TOKENS = 16         # from SKINNY_POLICY_TOKENS up to here the tcgen05 kernel; 16 = never:
# on row-major weights it reads 128-byte pieces of 128 rows per copy and stays below the library product
EPI_STORE, EPI_PARTIAL, EPI_SWIGLU = 0, 1, 2


def few_token_impl(T: int) -> str:
    """Which kernel takes a product of T tokens: "stream" / "regs" (mma.sync weight streamers), "tc5"
    (tcgen05 + TMA), or "" (none of the few-token kernels: the caller takes the library product)."""
    if skinny_impl == "tc5":
        return "tc5" if T <= max(TC5_POLICY_TOKENS, SKINNY_POLICY_TOKENS) else ""
    if T <= SKINNY_POLICY_TOKENS:
        # the streaming kernel is the faster one up to 8 tokens (one 8-token tile per row block); with two
        # tiles its stages shrink and the register-load kernel wins clearly (measured in whole decode steps)
        return "regs" if skinny_impl == "stream" and T > STREAM_POLICY_TOKENS else skinny_impl
    return "tc5" if T <= TC5_POLICY_TOKENS else ""


def stream_resident_shares(T: int, K: int) -> int:
    """For 9 to ``STREAM_RESIDENT_TOKENS`` tokens: the number of shares of K (one stage of the streamer each) with
    which the streaming kernel keeps the tokens resident, or 0 if this product is not taken that way."""
    if skinny_impl != "stream" or not (STREAM_POLICY_TOKENS < T <= min(16, STREAM_RESIDENT_TOKENS)):
        return 0
    chunks = (K + 1023) // 1024
    return chunks if chunks <= STREAM_RESIDENT_MAX_SHARES else 0


SWIGLU_FROM_SHARES_WIDE = True     # up to 8 tokens and a hidden size above two stages: gate/up as partial sums


def swiglu_shares(T: int, K: int, N: int) -> int:
    """The shares of K over which the stacked gate/up product [N, K] of T tokens leaves partial sums for
    ``swiglu_partial``, or 0 where the product's own SwiGLU epilogue is the better choice.  Partial sums pay
    where they keep the tokens' rows resident in the streamer: for 9 to 16 tokens, and for up to 8 tokens when
    K is wider than the rows the streamer keeps (the one-kernel form then copies the tokens with every stage)."""
    shares = stream_resident_shares(T, K)
    if shares:
        return shares
    chunks = (K + 1023) // 1024
    if SWIGLU_FROM_SHARES_WIDE and few_token_impl(T) == "stream" and T <= STREAM_POLICY_TOKENS and chunks > 2:
        sp = skinny_splits(N, K, T)
        if max(chunks * (i + 1) // sp - chunks * i // sp for i in range(sp)) <= 2:
            return sp
    return 0


def _impl_for(T: int, K: int, splits: int, epi: int) -> str:
    """The kernel one product runs on: ``few_token_impl`` by the number of tokens, and the streaming kernel for
    partial sums of 9 to 16 tokens over shares that keep the tokens resident."""
    impl = few_token_impl(T) or "tc5"
    if impl == "regs" and epi == EPI_PARTIAL and splits == stream_resident_shares(T, K):
        return "stream"
    return impl


def skinny_supported(x: torch.Tensor, w: torch.Tensor, limit: Optional[int] = None) -> bool:
    if limit is None:
        limit = max(TC5_POLICY_TOKENS, SKINNY_POLICY_TOKENS)
        if not few_token_impl(x.shape[0]):
            return False
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] <= limit
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def skinny_splits(N: int, K: int, T: int = 1, target_ctas: Optional[int] = None) -> int:
    """Shares of K over the grid: enough CTAs (16 rows of W each) for four per SM, every warp at
    least one group of 128 k.  The tcgen05 kernel has tiles of 128 rows and one CTA per SM."""
    impl = few_token_impl(T) or "tc5"
    if impl == "regs" and stream_resident_shares(T, K):
        return stream_resident_shares(T, K)
    if target_ctas is None:
        target_ctas = 4 * sm_count()
    if impl == "tc5":
        tiles = (N + 127) // 128
        return max(1, min((tc5_max_ctas() + tiles - 1) // tiles, ((K + 63) // 64) // 8, 16))
    tiles = (N + 15) // 16
    if impl == "stream":
        chunks = (K + 1023) // 1024          # the streaming kernel splits K in whole stages of 1024
        if T <= 8 and chunks > 2:
            # The kernel keeps the tokens in shared memory when no share of K is wider than two stages, and
            # a CTA then keeps one share for the whole launch: among the splits that allow it, take the one
            # whose busiest CTA reads least (rounds over the tiles x stages per share).
            best = None
            for sp in range((chunks + 1) // 2, min(chunks, 16) + 1):
                per_share = max(1, min(stream_max_ctas() // sp, tiles))
                widest = max(chunks * (i + 1) // sp - chunks * i // sp for i in range(sp))
                if widest > 2:
                    continue
                cost = -(-tiles // per_share) * widest
                if best is None or cost < best[0]:
                    best = (cost, sp)
            if best is not None:
                return best[1]
        return max(1, min((target_ctas + tiles - 1) // tiles, chunks, 16))
    groups = (K + 127) // 128
    return max(1, min((target_ctas + tiles - 1) // tiles, groups // 4, 16))


# Which few-token kernel runs: "stream" (persistent CTAs fed by bulk asynchronous copies,
# csrc/gemm_stream.cu) or "regs" (one wave of CTAs loading straight into registers, csrc/gemm_skinny.cu).
skinny_impl = "stream"
_FFN_FUSED = _os.environ.get("QD_FFN_FUSED", "1") != "0"      # gate/up and down of up to 8 tokens in one launch

_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """Multiprocessors of the (current) CUDA device: what grids of persistent CTAs and the splits of the
    attention kernels are sized by."""
    index = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    n = _sm_counts.get(index)
    if n is None:
        n = _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return n


def stream_max_ctas() -> int:
    """Two persistent CTAs of the weight streamer on every multiprocessor."""
    return 2 * sm_count()


def tc5_max_ctas() -> int:
    """The tcgen05 product runs one persistent CTA per multiprocessor."""
    return sm_count()


def tile_weight(w: torch.Tensor, halves: int = 1) -> torch.Tensor:
    """W [N, K] bfloat16 -> [ceil(N/128) * ceil(K/64), 128, 64], zero-padded, each tile stored as the
    shared-memory image the tensor cores read (rows of 128 bytes; the 16-byte piece c of row r sits at
    piece c ^ (r % 8): the 128-byte swizzle): ``gemm_tc5`` fetches a tile with one contiguous 16 KB copy.
    ``halves`` = 2 tiles the gate and the up half of a stacked [2F, K] matrix separately (gate tiles
    first), as the SwiGLU epilogue wants them."""
    N, K = w.shape
    parts = w.chunk(halves, dim=0)
    out = []
    for part in parts:
        n = part.shape[0]
        nt, kt = (n + 127) // 128, (K + 63) // 64
        padded = torch.zeros((nt * 128, kt * 64), dtype=w.dtype, device=w.device)
        padded[:n, :K] = part
        tiles = padded.view(nt, 128, kt, 64).permute(0, 2, 1, 3).contiguous().view(nt * kt, 128, 8, 8)
        r = torch.arange(128, device=w.device).view(128, 1)
        c = torch.arange(8, device=w.device).view(1, 8)
        src = (c ^ (r & 7)).view(1, 128, 8, 1).expand(tiles.shape[0], 128, 8, 8)    # piece at position p holds piece p ^ (r % 8)
        out.append(torch.gather(tiles, 2, src).view(nt * kt, 128, 64))
    return torch.cat(out, dim=0).contiguous()


def gemm_tc5_status() -> int:
    """0 unless a bounded wait inside the tcgen05 kernel ran out on the current device."""
    return int(library("gemm_tc5").qd_gemm_tc5_status())


def _skinny_call(x, w, bias, out, part, T, N, K, splits, epi, what, w_tiled=False):
    out_code = dtype_code(out.dtype) if out is not None else F32
    ldo = out.stride(0) if out is not None else 0
    impl = _impl_for(T, K, splits, epi)
    if impl == "tc5":
        _check(library("gemm_tc5").qd_gemm_tc5(
            _ptr(w), _ptr(x), _LL(x.stride(0)), _ptr(bias), _ptr(out), _I(out_code), _LL(ldo), _ptr(part),
            _I(T), _I(N), _I(K), _I(splits), _I(epi), _I(tc5_max_ctas()), _I(1 if w_tiled else 0), _stream()), what)
    elif impl == "stream":
        _check(library("gemm_stream").qd_gemm_stream(
            _ptr(w), _ptr(x), _LL(x.stride(0)), _ptr(bias), _ptr(out), _I(out_code), _LL(ldo), _ptr(part),
            _I(T), _I(N), _I(K), _I(splits), _I(epi), _I(stream_max_ctas()), _stream()), what)
    else:
        _check(library("gemm_skinny").qd_gemm_skinny(
            _ptr(w), _ptr(x), _LL(x.stride(0)), _ptr(bias), _ptr(out), _I(out_code), _LL(ldo), _ptr(part),
            _I(T), _I(N), _I(K), _I(splits), _I(epi), _stream()), what)


def gemm_stream_status() -> int:
    """0 unless a bounded wait inside the streaming kernel ran out on the current device."""
    return int(library("gemm_stream").qd_gemm_stream_status())


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[T, N] = x @ w^T (+ bias) for T <= 64, bfloat16 in, out bfloat16 or float32."""
    T, K = x.shape
    N = w.shape[0]
    assert skinny_supported(x, w, 1 << 30) and out.shape == (T, N) and out.stride(1) == 1
    _contig(w, "w")
    _skinny_call(x, w, bias, out, None, T, N, K, 1, EPI_STORE, "gemm_skinny")


def gemm_skinny_partial(x: torch.Tensor, w: torch.Tensor, splits: int) -> torch.Tensor:
    """float32 partial sums [splits, T, N] of x @ w^T over ``splits`` shares of K."""
    T, K = x.shape
    N = w.shape[0]
    assert skinny_supported(x, w, 1 << 30)
    _contig(w, "w")
    part = torch.empty((splits, T, N), dtype=torch.float32, device=x.device)
    _skinny_call(x, w, None, None, part, T, N, K, splits, EPI_PARTIAL, "gemm_skinny_partial")
    return part


def gemm_skinny_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[T, F] = silu(x @ Wg^T) * (x @ Wu^T) with w_gate_up = [Wg; Wu] of shape [2F, K]."""
    T, K = x.shape
    N = w_gate_up.shape[0]
    assert skinny_supported(x, w_gate_up, 1 << 30) and out.shape == (T, N // 2) and out.dtype == torch.bfloat16
    _contig(w_gate_up, "w"); _contig(out, "out")
    _skinny_call(x, w_gate_up, None, out, None, T, N, K, 1, EPI_SWIGLU, "gemm_skinny_swiglu")


def ffn_stream_supported(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor) -> bool:
    """Whether the one-launch feed-forward (gate/up + SwiGLU, a wait between CTAs, down) takes these sizes."""
    T, D = x.shape
    F = w_down.shape[1]
    return (_FFN_FUSED and T <= 8 and D <= 2048 and few_token_impl(T) == "stream" and skinny_supported(x, w_gate_up)
            and w_down.dtype == torch.bfloat16 and F % 8 == 0 and w_gate_up.shape[0] == 2 * F
            and w_down.shape[0] == D)


FFN_SYNC_WORDS = 64      # words of device memory a layer's one-launch feed-forward synchronises through


def ffn_stream(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, barrier: torch.Tensor,
               timeline: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 partial sums [splits, T, D] of (silu(x Wg^T) * (x Wu^T)) Wd^T for up to 8 tokens, in one
    launch of the weight streamer: between the two products a CTA waits for the others' columns of h that its
    share of the second product reads, its producer warp meanwhile fetches the second product's first weights.  ``barrier``: ``FFN_SYNC_WORDS`` int32 words
    on the device, zero before their first use, that belong to the caller (no two launches that may run
    at the same time share them); every launch leaves them ready for the next.  ``timeline``: for measurements,
    int64 [CTAs, 8] that takes the kernel's own nanosecond stamps."""
    assert barrier.dtype == torch.int32 and barrier.numel() >= FFN_SYNC_WORDS and barrier.is_cuda
    T, D = x.shape
    F = w_down.shape[1]
    _contig(w_gate_up, "w_gate_up"); _contig(w_down, "w_down")
    splits = skinny_splits(D, F, T)
    h = torch.empty((T, F), dtype=torch.bfloat16, device=x.device)
    part = torch.empty((splits, T, D), dtype=torch.float32, device=x.device)
    _check(library("gemm_stream").qd_ffn_stream(
        _ptr(w_gate_up), _ptr(x), _LL(x.stride(0)), _ptr(h), _LL(h.stride(0)), _ptr(w_down), _ptr(part), _I(T), _I(D),
        _I(F), _I(splits), _ptr(barrier), _I(stream_max_ctas()), _ptr(timeline), _stream()), "ffn_stream")
    return part


# ------------------------------------------------------------------- attention
def paged_attention_generic(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv: torch.Tensor,
                            block_table: torch.Tensor, token_req: torch.Tensor, positions: torch.Tensor,
                            n_tokens: int, H: int, G: int, d: int, page_size: int, scale: float,
                            window: int) -> None:
    """Attention of every token over keys 0..pos (or the last ``window`` of them) of its request,
    read from ``kv`` [pages, 2, G, page_size, d] through ``block_table`` [R, max_blocks].
    ``q`` points at the first query element; rows are ``q_stride`` elements apart."""
    assert block_table.dtype == torch.int32 and block_table.dim() == 2
    assert token_req.dtype == torch.int32 and positions.dtype == torch.int32
    assert out.shape == (n_tokens, H * d) and kv.dtype == q.dtype == out.dtype
    assert tuple(kv.shape[1:]) == (2, G, page_size, d)
    _contig(out, "out"); _contig(kv, "kv"); _contig(block_table, "block_table")
    _check(library("attention_generic").qd_paged_attention_generic(
        _ptr(q), _LL(q_stride), _ptr(out), _LL(out.stride(0)), _ptr(kv), _I(dtype_code(q.dtype)),
        _ptr(block_table), _I(block_table.shape[1]), _ptr(token_req), _ptr(positions), _I(n_tokens),
        _I(H), _I(G), _I(d), _I(page_size), _F(scale), _I(window), _stream()), "paged_attention_generic")


FLASH_HEAD_DIMS = (16, 32, 48, 64, 96, 128)


def flash_decode_supported(dtype, H: int, G: int, d: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and d in FLASH_HEAD_DIMS and H // G <= 16 and page_size % 16 == 0


def flash_prefill_supported(dtype, H: int, G: int, d: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and d in FLASH_HEAD_DIMS and H // G <= 64


_TICKETS = 1 << 16
_tickets = {}
# split-KV decode attention fed by TMA tensor copies at head sizes 64 and 128 (batch 64 at context 2,176: 43.0
# against 47.1 us a launch; QD_DECODE_TMA=0 keeps the cp.async kernel)
_DECODE_TMA = _os.environ.get("QD_DECODE_TMA", "1") != "0"


def decode_attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv: torch.Tensor,
                     block_table: torch.Tensor, token_req: torch.Tensor, positions: torch.Tensor,
                     n_tokens: int, H: int, G: int, d: int, page_size: int, scale: float, window: int,
                     splits: int, fused_combine: bool = True) -> None:
    """One query token per request over its cached keys (tensor cores, keys split over ``splits``
    CTAs per (request, kv head); partial results go through scratch memory when splits > 1)."""
    assert q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert out.shape == (n_tokens, H * d) and tuple(kv.shape[1:]) == (2, G, page_size, d)
    assert block_table.dtype == torch.int32 and block_table.dim() == 2
    _contig(out, "out"); _contig(kv, "kv"); _contig(block_table, "block_table")
    part_o = part_ml = tickets = None
    if splits > 1:
        part_o = torch.empty((n_tokens * H * splits, d), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n_tokens * H * splits, 2), dtype=torch.float32, device=q.device)
        if fused_combine and n_tokens * G <= _TICKETS:
            tickets = _tickets.get(q.device)
            if tickets is None:     # zero once; every launch leaves them zero again
                tickets = _tickets[q.device] = torch.zeros(_TICKETS, dtype=torch.int32, device=q.device)
    if _DECODE_TMA and d in (64, 128) and splits <= 64 and (splits == 1 or tickets is not None):
        # K/V chunks by TMA tensor copies instead of 16-byte cp.async
        _check(library("attention_flash").qd_decode_attention_tma(
            _ptr(q), _LL(q_stride), _ptr(out), _ptr(kv), _LL(kv.shape[0]), _ptr(block_table),
            _I(block_table.shape[1]), _ptr(token_req), _ptr(positions), _I(n_tokens), _I(H), _I(G), _I(d),
            _I(page_size), _F(scale), _I(window), _I(splits), _ptr(part_o), _ptr(part_ml), _ptr(tickets),
            _stream()), "decode_attention_tma")
        return
    _check(library("attention_flash").qd_decode_attention(
        _ptr(q), _LL(q_stride), _ptr(out), _ptr(kv), _ptr(block_table), _I(block_table.shape[1]),
        _ptr(token_req), _ptr(positions), _I(n_tokens), _I(H), _I(G), _I(d), _I(page_size), _F(scale),
        _I(window), _I(splits), _ptr(part_o), _ptr(part_ml), _ptr(tickets), _stream()), "decode_attention")


def decode_rope_supported(dtype: torch.dtype, H: int, G: int, d: int, page_size: int) -> bool:
    return (dtype == torch.bfloat16 and d in (16, 32, 48, 64, 96, 128) and H % G == 0 and H // G <= 16
            and page_size % 16 == 0)


def decode_attention_rope(part: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, kv: torch.Tensor,
                          block_table: torch.Tensor, token_req: torch.Tensor, positions: torch.Tensor,
                          slot_map: torch.Tensor, H: int, G: int, d: int, page_size: int, scale: float,
                          window: int, splits: int, write_kv: bool, rotary_dim: int, pairing: int,
                          cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                          timeline: Optional[torch.Tensor] = None) -> None:
    """One decoded token per request, from the float32 partial sums part [n_parts, T, (H+2G)*d] of q, k, v:
    bias, rotation by position, cache write and attention over the paged cache in one launch; the splits
    of a (token, kv head) combine through scratch memory, the last CTA to finish doing the sum."""
    n_parts, T, W = part.shape
    assert part.dtype == torch.float32 and W == (H + 2 * G) * d and out.shape == (T, H * d)
    assert out.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16 and tuple(kv.shape[1:]) == (2, G, page_size, d)
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and positions.dtype == torch.int32
    _contig(part, "part"); _contig(out, "out"); _contig(kv, "kv"); _contig(block_table, "block_table")
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == W
    part_o = part_ml = tickets = None
    if splits > 1:
        if T * G > _TICKETS:
            raise KernelError("decode_attention_rope: more (token, kv head) pairs than tickets")
        part_o = torch.empty((T * H * splits, d), dtype=torch.float32, device=part.device)
        part_ml = torch.empty((T * H * splits, 2), dtype=torch.float32, device=part.device)
        tickets = _tickets.get(part.device)
        if tickets is None:     # zero once; every launch leaves them zero again
            tickets = _tickets[part.device] = torch.zeros(_TICKETS, dtype=torch.int32, device=part.device)
    _check(library("attention_decode_rope").qd_decode_attention_rope(
        _ptr(part), _I(n_parts), _ptr(bias), _ptr(out), _ptr(kv), _ptr(block_table), _I(block_table.shape[1]),
        _ptr(token_req), _ptr(positions), _ptr(slot_map), _I(T), _I(H), _I(G), _I(d), _I(page_size), _F(scale),
        _I(window), _I(splits), _I(1 if write_kv else 0), _ptr(cos), _ptr(sin), _I(rotary_dim), _I(pairing),
        _ptr(part_o), _ptr(part_ml), _ptr(tickets), _ptr(timeline), _stream()),
        "decode_attention_rope")


def prefill_attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv: torch.Tensor,
                      block_table: torch.Tensor, cu_tokens: torch.Tensor, start_pos: torch.Tensor,
                      n_requests: int, n_tokens: int, H: int, G: int, d: int, page_size: int, scale: float,
                      window: int) -> None:
    """Portions of ``n_requests`` requests (tokens cu_tokens[r]..cu_tokens[r+1]-1 at positions
    start_pos[r]..) over their cached keys, causal, on tensor cores."""
    assert q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    # cu_tokens holds rows of q and out: they may start past row 0 (the rows before belong to another kernel)
    assert out.shape[0] >= n_tokens and out.shape[1] == H * d and tuple(kv.shape[1:]) == (2, G, page_size, d)
    assert block_table.dtype == torch.int32 and block_table.shape[0] >= n_requests
    assert cu_tokens.dtype == torch.int32 and start_pos.dtype == torch.int32
    _contig(out, "out"); _contig(kv, "kv"); _contig(block_table, "block_table")
    _check(library("attention_flash").qd_prefill_attention(
        _ptr(q), _LL(q_stride), _ptr(out), _ptr(kv), _ptr(block_table), _I(block_table.shape[1]),
        _ptr(cu_tokens), _ptr(start_pos), _I(n_requests), _I(n_tokens), _I(H), _I(G), _I(d), _I(page_size),
        _F(scale), _I(window), _stream()), "prefill_attention")


# -------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, draws: torch.Tensor,
           out: torch.Tensor) -> None:
    """out[r] = sampled token of logits[r] (float32 [R, V]); temperature 0 is argmax."""
    R, V = logits.shape
    assert logits.dtype == torch.float32 and temperature.dtype == torch.float32
    assert top_k.dtype == torch.int32 and draws.dtype == torch.float32 and out.dtype == torch.int32
    _contig(logits, "logits")
    _check(library("sampling").qd_sample(_ptr(logits), _I(R), _I(V), _ptr(temperature), _ptr(top_k),
                                         _ptr(draws), _ptr(out), _stream()), "sample")


def prefill_tc5_supported(dtype, H: int, G: int, d: int, page_size: int) -> bool:
    """What the tcgen05 prefill attention takes: bfloat16, head size 64 or 128, up to 16 query heads per KV
    head, pages of a multiple of 16 tokens."""
    return (dtype == torch.bfloat16 and d in (64, 128) and H % G == 0 and 1 <= H // G <= 16
            and page_size % 16 == 0)


def prefill_attention_tc5(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv: torch.Tensor,
                          block_table: torch.Tensor, cu_tokens: torch.Tensor, start_pos: torch.Tensor,
                          n_requests: int, n_tokens: int, H: int, G: int, d: int, page_size: int, scale: float,
                          window: int, timeline: Optional[torch.Tensor] = None) -> None:
    """``prefill_attention`` on tcgen05 tensor cores (accumulators in tensor memory, K/V tiles by TMA)."""
    assert q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert out.shape[0] >= n_tokens and out.shape[1] == H * d and tuple(kv.shape[1:]) == (2, G, page_size, d)
    assert block_table.dtype == torch.int32 and block_table.shape[0] >= n_requests
    assert cu_tokens.dtype == torch.int32 and start_pos.dtype == torch.int32
    _contig(out, "out"); _contig(kv, "kv"); _contig(block_table, "block_table")
    _check(library("attention_tc5").qd_prefill_attention_tc5(
        _ptr(q), _LL(q_stride), _ptr(out), _ptr(kv), _LL(kv.shape[0]), _ptr(block_table), _I(block_table.shape[1]),
        _ptr(cu_tokens), _ptr(start_pos), _I(n_requests), _I(n_tokens), _I(H), _I(G), _I(d), _I(page_size),
        _F(scale), _I(window), _ptr(timeline), _stream()), "prefill_attention_tc5")


def prefill_attention_tc5_status() -> int:
    """0, or which bounded wait of the tcgen05 attention kernel ran out since the last call (synchronises)."""
    return int(library("attention_tc5").qd_prefill_attention_tc5_status())


# library -> (its status function, its wait probe): the kernels with bounded waits on mbarriers or a grid barrier
_STATUS = {"gemm_stream": ("qd_gemm_stream_status", "qd_gemm_stream_wait_probe"),
           "gemm_tc5": ("qd_gemm_tc5_status", "qd_gemm_tc5_wait_probe"),
           "attention_tc5": ("qd_prefill_attention_tc5_status", "qd_prefill_attention_tc5_wait_probe"),
           "attention_flash": ("qd_decode_attention_tma_status", "qd_decode_attention_tma_wait_probe")}


def check_status() -> None:
    """Raise if a bounded wait inside one of the kernels with mbarrier or grid-barrier waits ran out since the
    last call: the results of that launch were void.  Synchronises the device; asks only the libraries this
    process has loaded; a status is reported once."""
    bad = []
    for name, (fn, _) in _STATUS.items():
        if _library_loaded(name):
            code = int(getattr(library(name), fn)())
            if code != 0:
                bad.append(f"{name} (status {code})")
    if bad:
        raise KernelError("a bounded wait ran out inside a kernel of " + ", ".join(bad) +
                          "; results of launches since the last check are invalid")


def wait_probe(name: str, poll_limit: int = 2048) -> None:
    """Launch library ``name``'s probe: one warp waits ``poll_limit`` polls, through the library's own wait
    function, on an mbarrier that nobody arrives at.  The wait runs out, the kernel ends, and the next
    ``check_status`` raises.  For tests of that chain; it harms nothing else."""
    _check(getattr(library(name), _STATUS[name][1])(ctypes.c_uint(poll_limit), _stream()), f"{name} wait probe")


# ------------------------------------------------------------------ latent attention
LATENT_MAX_RANK = 512


def latent_prep(u: torch.Tensor, q_off: int, q_rank: int, kv_off: int, r: int, dr: int, wq_norm: torch.Tensor,
                wkv_norm: torch.Tensor, eps: float, cos: torch.Tensor, sin: torch.Tensor, rot_dims: int,
                positions: torch.Tensor, slot_map: torch.Tensor, cq: torch.Tensor, cache: torch.Tensor,
                write_cache: bool) -> None:
    """From the float32 projections u [T, *]: cq [T, q_rank] = RMS norm of the query latent times its weight, and
    the cache row [normed latent (r) | rotated key part (dr)] written to each token's slot of ``cache``
    [pages, page_size, r + dr].  Norms and rotation in float32; ``rot_dims`` leading elements of the key part turn,
    pairs (2i, 2i + 1).  ``q_rank`` 0: there is no query latent (``cq`` is empty, ``wq_norm`` unused)."""
    T = u.shape[0]
    assert u.dtype == torch.float32 and u.stride(1) == 1 and cq.shape == (T, q_rank) and cq.dtype == cache.dtype
    assert cache.shape[-1] == r + dr and wq_norm.dtype == wkv_norm.dtype == torch.float32
    assert cos.dtype == torch.float32 and cos.shape[1] == rot_dims // 2 and positions.dtype == torch.int32
    _contig(cq, "cq"); _contig(cache, "cache")
    _check(library("latent_attention").qd_latent_prep(
        _ptr(u), _LL(u.stride(0)), _I(q_off), _I(q_rank), _I(kv_off), _I(r), _I(dr), _ptr(wq_norm), _ptr(wkv_norm),
        _F(eps), _ptr(cos), _ptr(sin), _I(rot_dims), _ptr(positions), _ptr(slot_map), _ptr(cq), _ptr(cache),
        _I(dtype_code(cache.dtype)), _I(1 if write_cache else 0), _I(T), _stream()), "latent_prep")


def latent_absorb(q: torch.Tensor, wuk: torch.Tensor, qcat: torch.Tensor, H: int, dn: int, dr: int, r: int,
                  cos: torch.Tensor, sin: torch.Tensor, rot_dims: int, positions: torch.Tensor,
                  pre: Optional[torch.Tensor] = None) -> None:
    """qcat[t, h] = [Wuk_h^T q_unrotated[t, h] (r) | rotate(q_rotated[t, h]) (dr)], float32; q float32
    [T, H * (dn + dr)], wuk [H * dn, r].  ``pre`` (float32 [H, T, r]): the first part, already made by a batched
    library product."""
    assert pre is None or (pre.dtype == torch.float32 and pre.shape == (H, q.shape[0], r) and pre.is_contiguous())
    T = q.shape[0]
    assert q.dtype == torch.float32 and q.shape == (T, H * (dn + dr)) and wuk.shape == (H * dn, r)
    assert qcat.dtype == torch.float32 and qcat.shape == (T, H, r + dr) and q.stride(1) == 1   # q: a column range is fine
    _contig(wuk, "wuk"); _contig(qcat, "qcat")
    _check(library("latent_attention").qd_latent_absorb(
        _ptr(q), _LL(q.stride(0)), _ptr(wuk), _I(dtype_code(wuk.dtype)), _ptr(qcat), _I(T), _I(H), _I(dn), _I(dr), _I(r), _ptr(cos),
        _ptr(sin), _I(rot_dims), _ptr(positions), _ptr(pre), _stream()), "latent_absorb")


def latent_attend(qcat: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, token_req: torch.Tensor,
                  positions: torch.Tensor, r: int, dr: int, page_size: int, scale: float, window: int, splits: int,
                  o_lat: torch.Tensor) -> None:
    """o_lat[t, h] = sum_j softmax_j(qcat[t, h] . row_j * scale) row_j[:r] over the cached rows j <= position of the
    token's request (``cache`` [pages, page_size, r + dr] through ``block_table``); float32 scores and weights;
    ``splits`` CTAs share a token's keys."""
    T, H, W = qcat.shape
    assert W == r + dr and o_lat.shape == (T, H, r) and o_lat.dtype == torch.float32 and qcat.dtype == torch.float32
    assert tuple(cache.shape[1:]) == (page_size, W) and block_table.dtype == torch.int32 and block_table.dim() == 2
    _contig(qcat, "qcat"); _contig(cache, "cache"); _contig(block_table, "block_table"); _contig(o_lat, "o_lat")
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((T * H * splits, r), dtype=torch.float32, device=qcat.device)
        part_ml = torch.empty((T * H * splits, 2), dtype=torch.float32, device=qcat.device)
    _check(library("latent_attention").qd_latent_attend(
        _ptr(qcat), _ptr(cache), _I(dtype_code(cache.dtype)), _ptr(block_table), _I(block_table.shape[1]),
        _ptr(token_req), _ptr(positions), _I(T), _I(H), _I(r), _I(dr), _I(page_size), _F(scale), _I(window),
        _I(splits), _ptr(o_lat), _ptr(part_o), _ptr(part_ml), _stream()), "latent_attend")
    if splits > 1:
        _launch_count[0] += 1


def latent_gather(cache: torch.Tensor, block_table: torch.Tensor, cu_tokens: torch.Tensor, start_pos: torch.Tensor,
                  n_requests: int, r: int, out: torch.Tensor, Lmax: int) -> None:
    """out[q * Lmax + j] = the first ``r`` elements of cached row j of request q, for every row of the request's context
    (what it holds and this step's tokens); rows past it are zero.  ``cache`` [pages, page_size, W]."""
    assert out.shape == (n_requests * Lmax, r) and out.dtype == cache.dtype and cache.dim() == 3
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.shape[0] >= n_requests
    _contig(cache, "cache"); _contig(block_table, "block_table"); _contig(out, "out")
    _check(library("latent_attention").qd_latent_gather(
        _ptr(cache), _I(dtype_code(cache.dtype)), _ptr(block_table), _I(block_table.shape[1]), _ptr(cu_tokens),
        _ptr(start_pos), _I(n_requests), _I(cache.shape[1]), _I(cache.shape[2]), _I(r), _ptr(out), _I(Lmax), _stream()),
        "latent_gather")


def round_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x rounded to bfloat16; x float32 [T, N] (a column range of a wider buffer is fine), out dense."""
    assert x.dtype == torch.float32 and out.dtype == torch.bfloat16 and x.shape == out.shape and x.stride(1) == 1
    _contig(out, "out")
    _check(library("latent_attention").qd_round_rows(_ptr(x), _LL(x.stride(0)), _ptr(out), _I(x.shape[0]),
                                                     _I(x.shape[1]), _stream()), "round_rows")


def latent_expand(o_lat: torch.Tensor, wuv: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor,
                  dv: int, pre: Optional[torch.Tensor] = None) -> None:
    """out[t, h * dv + i] = (Wuv_h o_lat[t, h])[i] * sigmoid(gate[t, h * dv + i]); gate float32 (a column slice of a
    wider buffer is fine) or None."""
    T, H, r = o_lat.shape
    assert wuv.shape == (H * dv, r) and out.shape == (T, H * dv) and out.dtype == wuv.dtype
    assert gate is None or (gate.dtype == torch.float32 and gate.shape == (T, H * dv) and gate.stride(1) == 1)
    # ``pre`` (float32 [H, T, dv]): Wuv_h o_lat[t, h] already made by a batched library product
    assert pre is None or (pre.dtype == torch.float32 and pre.shape == (H, T, dv) and pre.is_contiguous())
    _contig(o_lat, "o_lat"); _contig(wuv, "wuv"); _contig(out, "out")
    _check(library("latent_attention").qd_latent_expand(
        _ptr(o_lat), _ptr(wuv), _I(dtype_code(wuv.dtype)), _ptr(gate), _LL(gate.stride(0) if gate is not None else 0),
        _ptr(out), _I(dtype_code(out.dtype)), _I(T), _I(H), _I(dv), _I(r), _ptr(pre), _stream()), "latent_expand")


# ------------------------------------------------------------------ state-space mixer
def mamba_conv(u: torch.Tensor, x_off: int, C: int, taps: int, w: torch.Tensor, bias: torch.Tensor,
               state: torch.Tensor, conv_off: int, token_req: torch.Tensor, cu_tokens: torch.Tensor,
               slots: torch.Tensor, xbc: torch.Tensor, n_requests: int, update_state: bool) -> None:
    """xbc[t, c] = silu(bias[c] + sum_k w[c, k] * input[t - (taps - 1) + k, c]) over columns x_off.. of u (float32);
    inputs before a request's portion come from its state row (``state`` [slots, n], the last taps - 1 inputs at
    ``conv_off``, oldest first), which is then moved on by the portion when ``update_state``."""
    T = u.shape[0]
    assert u.dtype == torch.float32 and u.stride(1) == 1 and xbc.shape == (T, C) and xbc.dtype == torch.float32
    assert w.shape == (C, taps) and w.dtype == bias.dtype == torch.float32 and state.dtype == torch.float32
    _contig(w, "w"); _contig(xbc, "xbc"); _contig(state, "state")
    _check(library("mamba2").qd_mamba_conv(
        _ptr(u), _LL(u.stride(0)), _I(x_off), _I(C), _I(taps), _ptr(w), _ptr(bias), _ptr(state), _LL(state.stride(0)),
        _LL(conv_off), _ptr(token_req), _ptr(cu_tokens), _ptr(slots), _ptr(xbc), _I(T), _I(n_requests),
        _I(1 if update_state else 0), _stream()), "mamba_conv")
    if update_state and taps > 1 and u.shape[0] != n_requests:      # single tokens: the same launch moves the state on
        _launch_count[0] += 1


def mamba_scan(xbc: torch.Tensor, u: torch.Tensor, dt_off: int, dt_bias: torch.Tensor, A_log: torch.Tensor,
               D: torch.Tensor, state: torch.Tensor, cu_tokens: torch.Tensor, slots: torch.Tensor, y: torch.Tensor,
               n_requests: int, nh: int, P: int, N: int, G: int, write_state: bool = True) -> None:
    """The recurrence, request by request and head by head over the portion's tokens, float32:
    dt = softplus(u[t, dt_off + h] + dt_bias[h]); S <- exp(-exp(A_log[h]) dt) S + dt B x^T; y = S^T C + D[h] x, with
    xbc rows [x (nh * P) | B (G * N) | C (G * N)] and S [nh, P, N] at the start of the request's state row."""
    T = xbc.shape[0]
    assert xbc.dtype == u.dtype == y.dtype == state.dtype == torch.float32 and y.shape == (T, nh * P)
    assert xbc.shape[1] == nh * P + 2 * G * N and state.shape[1] >= nh * P * N
    _contig(xbc, "xbc"); _contig(y, "y"); _contig(state, "state")
    _check(library("mamba2").qd_mamba_scan(
        _ptr(xbc), _I(xbc.shape[1]), _ptr(u), _LL(u.stride(0)), _I(dt_off), _ptr(dt_bias), _ptr(A_log), _ptr(D),
        _ptr(state), _LL(state.stride(0)), _ptr(cu_tokens), _ptr(slots), _ptr(y), _I(n_requests), _I(nh), _I(P),
        _I(N), _I(G), _I(1 if write_state else 0), _stream()), "mamba_scan")


def mamba_gate_norm(y: torch.Tensor, u: torch.Tensor, z_off: int, w: torch.Tensor, out: torch.Tensor, groups: int,
                    eps: float) -> None:
    """out = v / sqrt(mean(v^2) + eps) * w over each of ``groups`` equal parts of v = y * silu(u[:, z_off:...])."""
    T, inner = y.shape
    assert y.dtype == u.dtype == w.dtype == torch.float32 and out.shape == (T, inner) and w.numel() == inner
    _contig(y, "y"); _contig(out, "out")
    _check(library("mamba2").qd_mamba_gate_norm(
        _ptr(y), _ptr(u), _LL(u.stride(0)), _I(z_off), _ptr(w), _ptr(out), _I(dtype_code(out.dtype)), _I(T),
        _I(inner), _I(groups), _F(eps), _stream()), "mamba_gate_norm")


# ------------------------------------------------------------------ routed experts
ACT_SILU, ACT_CLAMPED = 0, 1     # gated activations: silu(g) * u; the clamped gate (see ``gated_act``)
MOE_MAX_TOP = 32
MOE_ROUTE_TOP_SOFTMAX, MOE_ROUTE_SOFTMAX_ALL, MOE_ROUTE_TOP_SIGMOID = 0, 1, 2
MOE_FEW_ROWS = 8          # rows of one expert that the weight-streaming grouped product takes as one tile


def moe_tile_rows(n_pairs: int, E: int, K1: int, K2: int, dtype: torch.dtype) -> int:
    """Rows of one expert per CTA in the grouped products: 8 (each expert's weights streamed once past its few
    rows) while experts see about that many pairs or fewer, 64 (tensor-core tiles in bfloat16) when they see
    many, 16 otherwise and wherever the faster forms' 16-byte pieces do not fit."""
    per = 4 if dtype == torch.float32 else 8
    pieces_fit = K1 % per == 0 and K2 % per == 0
    if n_pairs <= MOE_FEW_ROWS * E and pieces_fit and MOE_FEW_ROWS * max(K1, K2) * (16 // per) <= 200 * 1024:
        return MOE_FEW_ROWS
    return 64 if n_pairs >= 32 * E else 16


def moe_route(h: torch.Tensor, wr: torch.Tensor, br: Optional[torch.Tensor], wsg: Optional[torch.Tensor], top: int,
              idx: torch.Tensor, wt: torch.Tensor, sgate: Optional[torch.Tensor], mode: int = MOE_ROUTE_TOP_SOFTMAX,
              correction: Optional[torch.Tensor] = None) -> None:
    """idx, wt [T, top] from the float32 logits wr h (+ br).  ``MOE_ROUTE_TOP_SOFTMAX``: the ``top`` largest logits and
    the softmax over those.  ``MOE_ROUTE_SOFTMAX_ALL``: scores = softmax over all outputs; the ``top`` largest of
    score + correction are chosen and weigh by their plain scores.  ``MOE_ROUTE_TOP_SIGMOID``: the ``top`` largest
    logits, each weighed by its own sigmoid.  sgate[t] = sigmoid(wsg . h[t]) when a shared expert's gate vector is
    given."""
    T, D = h.shape
    E = wr.shape[0]
    assert wr.shape == (E, D) and wr.dtype == h.dtype
    assert br is None or (br.dtype == torch.float32 and br.numel() == E)
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == E)
    assert idx.dtype == torch.int32 and wt.dtype == torch.float32 and idx.shape == wt.shape == (T, top)
    _contig(h, "h"); _contig(wr, "wr")
    logits = torch.empty((T, E), dtype=torch.float32, device=h.device)
    _check(library("moe").qd_moe_route(_ptr(h), _ptr(wr), _ptr(br), _ptr(wsg), _I(dtype_code(h.dtype)), _I(T), _I(D),
                                       _I(E), _I(top), _I(mode), _ptr(correction), _ptr(logits), _ptr(idx), _ptr(wt),
                                       _ptr(sgate), _stream()),
           "moe_route")
    _launch_count[0] += 1


def moe_choose(logits: torch.Tensor, top: int, idx: torch.Tensor, wt: torch.Tensor, mode: int = MOE_ROUTE_TOP_SOFTMAX,
               correction: Optional[torch.Tensor] = None) -> None:
    """The choice of ``moe_route`` from float32 logits [T, E] that a product left (they may be overwritten)."""
    T, E = logits.shape
    assert logits.dtype == torch.float32 and idx.dtype == torch.int32 and wt.dtype == torch.float32
    assert idx.shape == wt.shape == (T, top)
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == E)
    _contig(logits, "logits")
    _check(library("moe").qd_moe_topk(_ptr(logits), _I(T), _I(E), _I(top), _I(mode), _ptr(correction), _ptr(idx),
                                      _ptr(wt), _stream()), "moe_choose")


def moe_sort(idx: torch.Tensor, E: int, tile_rows: int, max_tiles: int, place: torch.Tensor, pair_at: torch.Tensor,
             meta: torch.Tensor, with_weights: Optional[int] = None) -> None:
    """Order the (token, choice) pairs by expert on the device: place[pair], pair_at[place], and ``meta`` =
    [offsets (E + 1) | number of tiles | (expert, first row, rows) per tile].  Only the first ``with_weights``
    experts (default: all) get row tiles: the others have no matrices (identity experts)."""
    n = idx.numel()
    assert place.numel() == n and pair_at.numel() == n and meta.numel() >= E + 2 + 3 * max_tiles
    _check(library("moe").qd_moe_sort(_ptr(idx), _I(n), _I(E), _I(E if with_weights is None else with_weights),
                                      _I(tile_rows), _I(max_tiles), _ptr(place), _ptr(pair_at), _ptr(meta), _stream()),
           "moe_sort")


def moe_gemm(a: torch.Tensor, pair_at: torch.Tensor, top: int, by_token: bool, w1: torch.Tensor,
             w2: Optional[torch.Tensor], out: torch.Tensor, meta: torch.Tensor, tile_rows: int, max_tiles: int,
             num_outputs: Optional[int] = None, act: int = ACT_SILU, limit: float = 0.0, alpha: float = 1.0,
             in_scale: Optional[torch.Tensor] = None) -> None:
    """Grouped product over the sorted pairs: out[place] = a_row W1[e]^T (or, with w2, act(a W1[e]^T, a W2[e]^T):
    silu(g) * u, or the clamped gate of ``gated_act``); a_row = a[token of the pair] when ``by_token`` else a[place];
    w [E, N, K].  ``num_outputs``: how many outputs the router has (``meta`` is laid out by it), if more than E.
    ``in_scale`` (float32, one per pair in the router's order): the pair's input row counts times this number, that
    is, its sums are multiplied by it before the gate."""
    E, N, K = w1.shape
    assert in_scale is None or (in_scale.dtype == torch.float32 and in_scale.is_contiguous())
    assert a.shape[1] == K and a.stride(1) == 1 and out.shape[1] == N and (w2 is None or w2.shape == w1.shape)
    _contig(w1, "w1"); _contig(out, "out")
    _check(library("moe").qd_moe_gemm(
        _ptr(a), _LL(a.stride(0)), _I(dtype_code(a.dtype)), _ptr(pair_at), _I(top), _I(1 if by_token else 0), _ptr(w1),
        _ptr(w2), _I(dtype_code(w1.dtype)), _ptr(out), _I(dtype_code(out.dtype)), _I(N), _I(K), _ptr(meta),
        _I(E if num_outputs is None else num_outputs), _I(tile_rows), _I(max_tiles), _I(1 if w2 is not None else 0),
        _I(act), _F(limit), _F(alpha), _ptr(in_scale), _stream()), "moe_gemm")


def moe_combine(y: torch.Tensor, place: torch.Tensor, wt: Optional[torch.Tensor], shared: Optional[torch.Tensor],
                sgate: Optional[torch.Tensor], out: torch.Tensor, idx: Optional[torch.Tensor] = None,
                with_weights: int = 0, h: Optional[torch.Tensor] = None, top: Optional[int] = None) -> None:
    """out[t] = sum_k wt[t, k] y[place[t, k]] + sgate[t] * shared[t] (shared [T, D], or float32 partial sums
    [n, T, D]; without ``sgate`` the shared expert counts in full); out float32.  With ``idx`` and ``h``: a pair
    whose expert index is ``with_weights`` or more is an identity expert and contributes wt * h[t].  ``wt`` None
    (then ``top`` says how many pairs a token has): the pairs' outputs are added as they are."""
    T, D = out.shape
    top = wt.shape[1] if wt is not None else int(top)
    assert y.dtype == torch.float32 and out.dtype == torch.float32 and y.shape[1] == D
    n_parts, stride = 1, 0
    if shared is not None:
        if shared.dim() == 3:
            n_parts, stride = shared.shape[0], T * D
            assert shared.dtype == torch.float32
        _contig(shared, "shared")
    if h is not None:
        assert idx is not None and idx.dtype == torch.int32 and h.shape == (T, D)
        _contig(h, "h")
    _check(library("moe").qd_moe_combine(
        _ptr(y), _ptr(place), _ptr(wt), _I(top), _ptr(shared), _I(dtype_code(shared.dtype) if shared is not None else 0),
        _I(n_parts), _LL(stride), _ptr(sgate), _ptr(out), _I(T), _I(D), _ptr(idx if h is not None else None),
        _I(with_weights), _ptr(h), _I(dtype_code(h.dtype) if h is not None else 0), _stream()), "moe_combine")


# ------------------------------------------------------------------ gated branches, short convolutions
def gated_add_norm(x: torch.Tensor, delta: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                   weight: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, eps: float = 0.0,
                   rows: Optional[torch.Tensor] = None, write_back: bool = True,
                   gate_bias: Optional[torch.Tensor] = None) -> None:
    """x += sigmoid(gate + gate_bias) * delta, element by element (x float32 [T, D]; gate float32 logits [T, D] or None,
    gate_bias float32 [D] or None; delta
    [T, D], or float32 partial sums [n, T, D]); with ``weight`` also out[r] = x[s] / sqrt(mean(x[s]^2) + eps) * weight,
    s = rows[r] (or r).  ``write_back`` False leaves x as it was (the norm still sees the sum)."""
    T, D = x.shape
    assert x.dtype == torch.float32 and (gate is None or (gate.dtype == torch.float32 and gate.shape == x.shape))
    _contig(x, "x")
    n_parts = 1
    if delta is not None:
        if delta.dim() == 3:
            n_parts = delta.shape[0]
            assert delta.dtype == torch.float32 and tuple(delta.shape[1:]) == (T, D)
        else:
            assert delta.shape == x.shape
        _contig(delta, "delta")
    if gate is not None:
        _contig(gate, "gate")
    assert gate_bias is None or (gate is not None and gate_bias.dtype == torch.float32 and gate_bias.numel() == D
                                 and gate_bias.is_contiguous())
    n_rows = T
    if weight is not None:
        n_rows = out.shape[0]
        assert weight.dtype == torch.float32 and weight.numel() == D and out.shape[1] == D and out.is_contiguous()
        assert rows is None or (rows.dtype == torch.int32 and rows.numel() == n_rows)
    _check(library("gated_block").qd_gated_add_norm(
        _ptr(x), _ptr(delta), _I(dtype_code(delta.dtype) if delta is not None else 0), _I(n_parts), _LL(T * D),
        _ptr(gate), _ptr(gate_bias), _ptr(weight), _ptr(out), _I(dtype_code(out.dtype) if out is not None else 0),
        _ptr(rows),
        _I(n_rows), _I(D), _F(eps), _I(1 if write_back else 0), _stream()), "gated_add_norm")


def short_conv(u: torch.Tensor, w: torch.Tensor, state: Optional[torch.Tensor], state_off: int,
               token_req: torch.Tensor, cu_tokens: torch.Tensor, slots: torch.Tensor, out: torch.Tensor,
               n_requests: int, residual: bool, update_state: bool) -> None:
    """out[t, c] = (u[t, c] if ``residual``) + sum_j w[c, j] u[t - taps + 1 + j, c] within each request of the flat
    batch; inputs before a portion come from the request's row of ``state`` (float32 [slots, n]; this convolution's
    (taps - 1) x C kept inputs, oldest first, at ``state_off``), which is moved on by the portion when
    ``update_state``.  u [T, C] (a column range is fine), w float32 [C, taps]."""
    T, C = u.shape
    taps = w.shape[1]
    assert w.shape == (C, taps) and w.dtype == torch.float32 and w.is_contiguous() and u.stride(1) == 1
    assert out.shape == (T, C) and out.stride(1) == 1
    assert taps == 1 or (state is not None and state.dtype == torch.float32 and state.is_contiguous())
    _check(library("gated_block").qd_short_conv(
        _ptr(u), _I(dtype_code(u.dtype)), _LL(u.stride(0)), _I(C), _I(taps), _ptr(w), _ptr(state),
        _LL(state.stride(0) if state is not None else 0), _LL(state_off), _ptr(token_req), _ptr(cu_tokens), _ptr(slots),
        _ptr(out), _I(dtype_code(out.dtype)), _LL(out.stride(0)), _I(T), _I(n_requests), _I(1 if residual else 0),
        _I(1 if update_state else 0), _stream()), "short_conv")
    if update_state and taps > 1 and u.shape[0] != n_requests:      # single tokens: the same launch moves the state on
        _launch_count[0] += 1


def concat_round(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = [a[t] | b[t]] in out's dtype; a, b float32 [T, D]."""
    T, D = a.shape
    assert a.dtype == b.dtype == torch.float32 and b.shape == a.shape and out.shape == (T, 2 * D)
    _contig(a, "a"); _contig(b, "b"); _contig(out, "out")
    _check(library("gated_block").qd_concat_round(_ptr(a), _ptr(b), _ptr(out), _I(dtype_code(out.dtype)), _I(T), _I(D),
                                                  _stream()), "concat_round")


ACT_GELU_TANH = 0       # plain (ungated) activations of ``plain_act``


def plain_act(z: torch.Tensor, out: torch.Tensor, act: int = ACT_GELU_TANH) -> None:
    """out = act(z) element by element; z float32 [T, F], or float32 partial sums [n, T, F] that are added up first."""
    n_parts = z.shape[0] if z.dim() == 3 else 1
    assert z.dtype == torch.float32 and tuple(z.shape[-2:]) == tuple(out.shape)
    _contig(z, "z"); _contig(out, "out")
    _check(library("gated_block").qd_plain_act(_ptr(z), _I(n_parts), _LL(out.numel()), _ptr(out),
                                               _I(dtype_code(out.dtype)), _LL(out.numel()), _I(act), _stream()),
           "plain_act")


# ------------------------------------------------------------------ differential attention
def diff_conv_write(u: torch.Tensor, H: int, G: int, d: int, vd: int, w: Optional[torch.Tensor],
                    state: Optional[torch.Tensor], state_off: int, token_req: torch.Tensor, cu_tokens: torch.Tensor,
                    slots: torch.Tensor, q_out: torch.Tensor, kv: torch.Tensor, slot_map: torch.Tensor, page_size: int,
                    n_requests: int, write: bool) -> None:
    """The stacked projection u (float32 [T, >= C], C = H * 2d + G * 2d + G * vd) through a short causal convolution
    per channel (w float32 [C, taps], or None for none; the kept inputs in the requests' rows of ``state`` at
    ``state_off``): q_out [T, H * 2d] dense, keys and values to each token's slot of the paged cache ``kv`` (a page:
    keys [G, page_size, 2d], then values [G, page_size, vd]).  With ``write`` the cache is written and the state
    moved on."""
    T = u.shape[0]
    C = H * 2 * d + G * 2 * d + G * vd
    taps = w.shape[1] if w is not None else 0
    assert u.dtype == torch.float32 and u.stride(1) == 1 and u.shape[1] >= C
    assert w is None or (w.shape == (C, taps) and w.dtype == torch.float32 and w.is_contiguous())
    assert q_out.shape == (T, H * 2 * d) and q_out.dtype == kv.dtype
    assert taps <= 1 or (state is not None and state.dtype == torch.float32 and state.is_contiguous())
    _contig(q_out, "q_out"); _contig(kv, "kv")
    _check(library("attention_diff").qd_diff_conv_write(
        _ptr(u), _LL(u.stride(0)), _I(H), _I(G), _I(d), _I(vd), _I(taps), _ptr(w), _ptr(state),
        _LL(state.stride(0) if state is not None else 0), _LL(state_off), _ptr(token_req), _ptr(cu_tokens), _ptr(slots),
        _ptr(q_out), _ptr(kv), _I(dtype_code(kv.dtype)), _ptr(slot_map), _I(page_size), _I(T), _I(n_requests),
        _I(1 if write else 0), _stream()), "diff_conv_write")
    if write and taps > 1 and T != n_requests:      # single tokens: the same launch moves the state on
        _launch_count[0] += 1


def diff_attention_generic(q: torch.Tensor, out: torch.Tensor, kv: torch.Tensor, block_table: torch.Tensor,
                           token_req: torch.Tensor, positions: torch.Tensor, H: int, G: int, d: int, vd: int,
                           page_size: int, scale: float, cap: float, lam: float, eps: float, out_scale: float,
                           window: int, gate: Optional[torch.Tensor]) -> None:
    """Differential attention, one warp per (token, head), float32 arithmetic, any sizes: two softmax maps over the
    same values, o = a1 - lam * a2, divided by its root mean square over the head, times ``out_scale`` and
    sigmoid(gate[t, h]).  q [T, H * 2d], out [T, H * vd] in the cache's dtype; gate float32 [T, H] logits (a column
    range of a wider buffer is fine) or None."""
    T = q.shape[0]
    assert q.shape == (T, H * 2 * d) and out.shape == (T, H * vd) and q.dtype == out.dtype == kv.dtype
    assert gate is None or (gate.dtype == torch.float32 and gate.shape == (T, H) and gate.stride(1) == 1)
    _contig(q, "q"); _contig(out, "out"); _contig(kv, "kv"); _contig(block_table, "block_table")
    _check(library("attention_diff").qd_diff_attention_generic(
        _ptr(q), _ptr(out), _ptr(kv), _I(dtype_code(kv.dtype)), _ptr(block_table), _I(block_table.shape[1]),
        _ptr(token_req), _ptr(positions), _I(T), _I(H), _I(G), _I(d), _I(vd), _I(page_size), _F(scale), _F(cap),
        _F(lam), _F(eps), _F(out_scale), _I(window), _ptr(gate), _LL(gate.stride(0) if gate is not None else 0),
        _stream()), "diff_attention_generic")


DIFF_MAX_VDIM = 512


DIFF_MMA_PAIRS = 32      # (token, head within the group) pairs of one tile of the tensor-core kernel (two rows each)
DIFF_MMA = _os.environ.get("QD_DIFF_MMA", "1") != "0"      # 0: every dtype and size on the float32 kernel


def diff_mma_supported(dtype: torch.dtype, H: int, G: int, d: int, vd: int) -> bool:
    """What the tensor-core form of the differential attention takes: bfloat16, per-map key sizes and value sizes
    that are multiples of 8 up to 128, groups of up to 32 query heads per key/value head; any page size."""
    return (dtype == torch.bfloat16 and H % G == 0 and H // G <= DIFF_MMA_PAIRS and d % 8 == 0 and vd % 8 == 0
            and 0 < d <= 128 and 0 < vd <= 128)


def diff_attention_mma(q: torch.Tensor, out: torch.Tensor, kv: torch.Tensor, block_table: torch.Tensor,
                       cu_tokens: torch.Tensor, start_pos: torch.Tensor, n_requests: int, n_tokens: int, H: int, G: int,
                       d: int, vd: int, page_size: int, scale: float, cap: float, lam: float, eps: float,
                       out_scale: float, window: int, gate: Optional[torch.Tensor], splits: int = 1) -> None:
    """``diff_attention_generic`` on tensor cores for portions of ``n_requests`` requests (rows cu_tokens[r] ..
    cu_tokens[r+1]-1 of q and out, at positions start_pos[r]..): a decoded token is a portion of one.  ``splits`` > 1
    shares every tile's keys among that many CTAs (for steps of few tokens over long contexts); a second launch adds
    their parts up."""
    assert q.dtype == out.dtype == kv.dtype == torch.bfloat16 and q.shape[1] == H * 2 * d and out.shape[1] == H * vd
    assert kv.numel() % (G * page_size * (2 * d + vd)) == 0
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.shape[0] >= n_requests
    assert cu_tokens.dtype == torch.int32 and start_pos.dtype == torch.int32
    assert gate is None or (gate.dtype == torch.float32 and gate.shape[1] == H and gate.stride(1) == 1)
    _contig(q, "q"); _contig(out, "out"); _contig(kv, "kv"); _contig(block_table, "block_table")
    ntok = DIFF_MMA_PAIRS // (H // G)
    tiles = n_tokens // ntok + n_requests            # at least sum over requests of ceil(tokens / ntok)
    part_o = part_ml = None
    if splits > 1:
        rows = out.shape[0] * H * 2
        part_o = torch.empty((rows * splits, vd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((rows * splits, 2), dtype=torch.float32, device=q.device)
    _check(library("attention_diff").qd_diff_attention_mma(
        _ptr(q), _ptr(out), _ptr(kv), _ptr(block_table), _I(block_table.shape[1]), _ptr(cu_tokens), _ptr(start_pos),
        _I(n_requests), _I(n_tokens), _I(tiles), _I(H), _I(G), _I(d), _I(vd), _I(page_size), _F(scale), _F(cap),
        _F(lam), _F(eps), _F(out_scale), _I(window), _ptr(gate), _LL(gate.stride(0) if gate is not None else 0),
        _I(splits), _ptr(part_o), _ptr(part_ml), _stream()), "diff_attention_mma")
    if splits > 1:
        _launch_count[0] += 1


def diff_decode_splits(ctas_without_split: int, max_keys: int) -> int:
    """CTAs per (token, KV head) of the tensor-core kernel for single tokens: as many as fill two CTAs on every
    multiprocessor, none with fewer than one tile of 64 keys, at most 64."""
    by_fill = max(1, 2 * sm_count() // max(1, ctas_without_split))
    by_work = max(1, (max_keys + 63) // 64)
    return max(1, min(by_fill, by_work, 64))


def diff_attention(q: torch.Tensor, out: torch.Tensor, kv: torch.Tensor, ctx, group, H: int, G: int, d: int, vd: int,
                   scale: float, cap: float, lam: float, eps: float, out_scale: float, window: int,
                   gate: Optional[torch.Tensor]) -> None:
    """Differential attention for the step ``ctx`` over the paged cache of ``group``: the kernel for these sizes.
    Single tokens (all of the step, or the first ``num_decode`` of a mixed one) share their keys among CTAs."""
    if not (DIFF_MMA and diff_mma_supported(q.dtype, H, G, d, vd)):
        diff_attention_generic(q, out, kv, group.block_table, ctx.token_request, ctx.positions, H, G, d, vd,
                               group.page_size, scale, cap, lam, eps, out_scale, window, gate)
        return
    T = q.shape[0]
    args = (H, G, d, vd, group.page_size, scale, cap, lam, eps, out_scale, window, gate)
    nd = T if ctx.all_decode else getattr(ctx, "num_decode", 0)
    if nd:
        keys = ctx.max_context if ctx.all_decode else ctx.decode_max_context
        splits = diff_decode_splits(nd * G, min(keys, window or keys))
        diff_attention_mma(q, out, kv, group.block_table, ctx.cu_tokens, ctx.start_pos, nd, nd, *args, splits=splits)
    if nd < T:
        diff_attention_mma(q, out, kv, group.block_table[nd:], ctx.cu_tokens[nd:], ctx.start_pos[nd:],
                           ctx.num_requests - nd, T - nd, *args)


# ------------------------------------------------------------------ tanh norm, gated activations, token gate
def add_tanh_norm(x: torch.Tensor, addends, norms, rows: Optional[torch.Tensor] = None, write_back: bool = True,
                  copy_out: Optional[torch.Tensor] = None) -> None:
    """One launch over the rows of the residual sum x (float32 [T, D]): v = x + the pending ``addends``; x = v when
    ``write_back``; every norm (w, b, alpha, out) of ``norms`` writes out = tanh(alpha v) w + b; ``copy_out`` gets v
    itself in its own dtype.  ``addends``: up to two of (tensor [T, D] or float32 partial sums [n, T, D], unit) where
    unit is None or (u float32 [D], eps): the addend then joins as a / sqrt(mean(a^2) + eps) * u; a third element
    ``mult`` multiplies the addend by a constant.  A norm given as ("rms", w, eps, out) writes
    out = v / sqrt(mean(v^2) + eps) * w instead of the tanh form.  ``rows`` (int32): only these rows, outputs in their
    order."""
    T, D = x.shape
    assert x.dtype == torch.float32 and len(addends) <= 2 and len(norms) <= 2
    _contig(x, "x")
    n_rows = T if rows is None else rows.numel()
    args = [_ptr(x), _I(T), _I(D)]
    for k in range(2):
        if k < len(addends):
            a, unit = addends[k][:2]
            mult = float(addends[k][2]) if len(addends[k]) > 2 else 1.0
            parts = a.shape[0] if a.dim() == 3 else 1
            assert tuple(a.shape[-2:]) == (T, D) and (parts == 1 or a.dtype == torch.float32)
            _contig(a, "addend")
            uw, ue = unit if unit is not None else (None, 0.0)
            assert uw is None or (uw.dtype == torch.float32 and uw.numel() == D)
            args += [_ptr(a), _I(dtype_code(a.dtype)), _I(parts), _ptr(uw), _F(ue), _F(mult)]
        else:
            args += [_ptr(None), _I(0), _I(1), _ptr(None), _F(0.0), _F(1.0)]
    for k in range(2):
        if k < len(norms) and isinstance(norms[k][0], str):
            _, w, eps, out = norms[k]
            assert w.dtype == torch.float32 and w.numel() == D and out.shape == (n_rows, D)
            _contig(out, "out")
            args += [_ptr(w), _ptr(None), _F(0.0), _ptr(out), _I(dtype_code(out.dtype)), _I(1), _F(eps)]
        elif k < len(norms):
            w, b, alpha, out = norms[k]
            assert w.dtype == b.dtype == torch.float32 and w.numel() == b.numel() == D and out.shape == (n_rows, D)
            _contig(out, "out")
            args += [_ptr(w), _ptr(b), _F(alpha), _ptr(out), _I(dtype_code(out.dtype)), _I(0), _F(0.0)]
        else:
            args += [_ptr(None), _ptr(None), _F(0.0), _ptr(None), _I(0), _I(0), _F(0.0)]
    if copy_out is not None:
        assert copy_out.shape == (n_rows, D)
        _contig(copy_out, "copy_out")
    args += [_ptr(rows), _I(n_rows), _I(1 if write_back else 0), _ptr(copy_out),
             _I(dtype_code(copy_out.dtype) if copy_out is not None else 0), _stream()]
    _check(library("norm_act").qd_add_tanh_norm(*args), "add_tanh_norm")


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, act: int = ACT_SILU, limit: float = 0.0,
              alpha: float = 1.0) -> None:
    """out[t, f] = act(g, u), g = gate_up[t, f], u = gate_up[t, F + f].  ``ACT_SILU``: silu(g) * u.  ``ACT_CLAMPED``:
    g' = min(g, limit), u' = clamp(u, -limit, limit), g' * sigmoid(alpha * g') * (u' + 1)."""
    T, F = out.shape
    assert gate_up.shape == (T, 2 * F)
    _contig(gate_up, "gate_up"); _contig(out, "out")
    _check(library("norm_act").qd_gated_act(_ptr(gate_up), _I(dtype_code(gate_up.dtype)), _ptr(out),
                                            _I(dtype_code(out.dtype)), _I(T), _I(F), _I(act), _F(limit), _F(alpha),
                                            _stream()), "gated_act")


def token_gate(z: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, j] = gelu_tanh(z[t, j]) * table[tokens[t], j]; z, out [T, W], table [vocab, W]."""
    T, W = z.shape
    assert out.shape == (T, W) and table.shape[1] == W and tokens.dtype == torch.int32
    _contig(z, "z"); _contig(table, "table"); _contig(out, "out")
    _check(library("norm_act").qd_token_gate(_ptr(z), _I(dtype_code(z.dtype)), _ptr(table), _I(dtype_code(table.dtype)),
                                             _ptr(tokens), _ptr(out), _I(dtype_code(out.dtype)), _I(T), _I(W),
                                             _stream()), "token_gate")


# ------------------------------------------------------------------ attention with a sink
def qk_norm_rope_write(qkv: torch.Tensor, H: int, G: int, d: int, vd: int, wq: Optional[torch.Tensor],
                       wk: Optional[torch.Tensor], eps: float, rotary_dim: int, pairing: int,
                       cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor,
                       q_out: torch.Tensor, kv: torch.Tensor, slot_map: torch.Tensor, page_size: int, write_kv: bool,
                       v_source: Optional[torch.Tensor] = None, lam: Optional[torch.Tensor] = None) -> None:
    """From qkv [T, H*d + G*d + G*vd] (float32 or bfloat16): q and k unit-normalised per head times wq / wk (float32
    [d]; None: no norm), their first ``rotary_dim`` elements turned by the table rows of ``positions``; q to q_out
    [T, H*d], k and v to the token's slot of ``kv`` (pages of [G, page_size, d] keys then [G, page_size, vd] values).
    With ``v_source`` ([T, G*vd], rows may be strided; same dtype as qkv) and ``lam`` (float32, one number on the
    device): the values written are (1 - lam) v + lam v_source."""
    T = qkv.shape[0]
    assert qkv.shape[1] == H * d + G * d + G * vd and qkv.stride(1) == 1 and positions.dtype == torch.int32
    assert q_out.shape == (T, H * d) and q_out.is_contiguous()
    assert (wq is None) == (wk is None) and (wq is None or (wq.dtype == wk.dtype == torch.float32 and wq.numel() == d))
    if rotary_dim:
        assert cos.dtype == sin.dtype == torch.float32 and cos.shape[1] == rotary_dim // 2
    if write_kv:
        assert kv.numel() % (G * page_size * (d + vd)) == 0 and slot_map.dtype == torch.int32
        _contig(kv, "kv")
    if v_source is not None:
        assert v_source.dtype == qkv.dtype and v_source.shape == (T, G * vd) and v_source.stride(1) == 1
        assert lam is not None and lam.dtype == torch.float32 and lam.numel() == 1
    _check(library("attention_sink").qd_qk_norm_rope_write(
        _ptr(qkv), _I(dtype_code(qkv.dtype)), _LL(qkv.stride(0)), _I(T), _I(H), _I(G), _I(d), _I(vd), _ptr(wq), _ptr(wk),
        _F(eps), _I(rotary_dim), _I(pairing), _ptr(cos), _ptr(sin), _ptr(positions), _ptr(q_out),
        _I(dtype_code(q_out.dtype)), _ptr(kv), _I(dtype_code(kv.dtype)), _ptr(slot_map), _I(page_size),
        _I(1 if write_kv else 0), _ptr(v_source), _LL(v_source.stride(0) if v_source is not None else 0), _ptr(lam),
        _stream()), "qk_norm_rope_write")


def sink_attention_generic(q: torch.Tensor, out: torch.Tensor, kv: torch.Tensor, block_table: torch.Tensor,
                           token_req: torch.Tensor, positions: torch.Tensor, H: int, G: int, d: int, vd: int,
                           page_size: int, scale: float, window: int, sinks: Optional[torch.Tensor], chunk: int = 0,
                           gate: Optional[torch.Tensor] = None, out_scale: float = 1.0) -> None:
    """Attention of every token over keys 0..pos (or the last ``window``; with ``chunk`` only those of the query's
    own block of ``chunk`` positions) of its request with a sink in the softmax's denominator (``sinks`` float32 [H],
    or None), values of size ``vd``; q [T, H*d], out [T, H*vd] (rows may be strided: a column range of a wider
    tensor); head h's output is multiplied by ``out_scale`` and, with ``gate`` (float32 [T, >= H] logits, rows may be
    strided), by sigmoid(gate[t, h]); float32 arithmetic, any sizes."""
    T = q.shape[0]
    assert q.shape == (T, H * d) and out.shape == (T, H * vd) and q.dtype == out.dtype == kv.dtype
    assert q.stride(1) == 1 and out.stride(1) == 1
    assert gate is None or (gate.dtype == torch.float32 and gate.shape[0] == T and gate.stride(1) == 1)
    assert kv.numel() % (G * page_size * (d + vd)) == 0
    assert block_table.dtype == torch.int32 and block_table.dim() == 2
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == H)
    _contig(kv, "kv"); _contig(block_table, "block_table")
    _check(library("attention_sink").qd_sink_attention_generic(
        _ptr(q), _LL(q.stride(0)), _ptr(out), _LL(out.stride(0)), _ptr(kv), _I(dtype_code(q.dtype)), _ptr(block_table),
        _I(block_table.shape[1]), _ptr(token_req), _ptr(positions), _I(T), _I(H), _I(G), _I(d), _I(vd), _I(page_size),
        _F(scale), _I(window), _ptr(sinks), _I(chunk), _ptr(gate), _LL(gate.stride(0) if gate is not None else 0),
        _F(out_scale), _stream()), "sink_attention_generic")


SINK_MMA_ROWS = 64       # rows, (token, head within the group) pairs, of one tile of the tensor-core kernel


def sink_mma_supported(dtype: torch.dtype, H: int, G: int, d: int, vd: int) -> bool:
    """What the tensor-core form of the sink attention takes: bfloat16, head sizes that are multiples of 8 up to 128,
    groups of up to 64 query heads per key/value head; any page size."""
    return (dtype == torch.bfloat16 and H % G == 0 and H // G <= SINK_MMA_ROWS and d % 8 == 0 and vd % 8 == 0
            and 0 < d <= 128 and 0 < vd <= 128)


def sink_attention_mma(q: torch.Tensor, out: torch.Tensor, kv: torch.Tensor, block_table: torch.Tensor,
                       cu_tokens: torch.Tensor, start_pos: torch.Tensor, n_requests: int, n_tokens: int, H: int, G: int,
                       d: int, vd: int, page_size: int, scale: float, window: int, sinks: Optional[torch.Tensor],
                       splits: int = 1, chunk: int = 0, gate: Optional[torch.Tensor] = None,
                       out_scale: float = 1.0) -> None:
    """``sink_attention_generic`` on tensor cores for portions of ``n_requests`` requests (rows cu_tokens[r] ..
    cu_tokens[r+1]-1 of q and out, at positions start_pos[r]..): a decoded token is a portion of one.  ``splits`` > 1
    shares every tile's keys among that many CTAs (for steps of few tokens over long contexts).  ``chunk``, ``gate``,
    ``out_scale`` and strided rows of ``out`` as for the generic kernel."""
    assert q.dtype == out.dtype == kv.dtype == torch.bfloat16 and q.shape[1] == H * d and out.shape[1] == H * vd
    assert out.stride(1) == 1 and out.stride(0) % 2 == 0
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1)
    assert kv.numel() % (G * page_size * (d + vd)) == 0
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.shape[0] >= n_requests
    assert cu_tokens.dtype == torch.int32 and start_pos.dtype == torch.int32
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == H)
    _contig(q, "q"); _contig(kv, "kv"); _contig(block_table, "block_table")
    ntok = SINK_MMA_ROWS // (H // G)
    tiles = n_tokens // ntok + n_requests            # at least sum over requests of ceil(tokens / ntok)
    part_o = part_ml = tickets = None
    if splits > 1:
        rows = out.shape[0] * H
        part_o = torch.empty((rows * splits, vd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((rows * splits, 2), dtype=torch.float32, device=q.device)
        if tiles * G <= _TICKETS:
            tickets = _tickets.get(q.device)
            if tickets is None:     # zero once; every launch leaves them zero again
                tickets = _tickets[q.device] = torch.zeros(_TICKETS, dtype=torch.int32, device=q.device)
    _check(library("attention_sink").qd_sink_attention_mma(
        _ptr(q), _ptr(out), _ptr(kv), _ptr(block_table), _I(block_table.shape[1]), _ptr(cu_tokens), _ptr(start_pos),
        _I(n_requests), _I(n_tokens), _I(tiles), _I(H), _I(G), _I(d), _I(vd), _I(page_size), _F(scale), _I(window),
        _ptr(sinks), _I(splits), _ptr(part_o), _ptr(part_ml), _ptr(tickets), _I(chunk), _ptr(gate),
        _LL(gate.stride(0) if gate is not None else 0), _F(out_scale), _LL(out.stride(0)), _stream()),
        "sink_attention_mma")
    if splits > 1 and tickets is None:
        _launch_count[0] += 1


# ------------------------------------------------------------------ between the q/k/v product and attention
QKV_NORMS = {"none": 0, "whole": 1, "head": 2}


def qkv_prep(u: torch.Tensor, H: int, G: int, d: int, vd: int, conv_w: Optional[torch.Tensor],
             state: Optional[torch.Tensor], state_off: int, ctx, update_state: bool, norm: str, norm_after: bool,
             wq: Optional[torch.Tensor], wk: Optional[torch.Tensor], eps: float, rotary_dim: int, pairing: int,
             cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], q_out: torch.Tensor, kv: torch.Tensor,
             slot_map: torch.Tensor, page_size: int, write_kv: bool) -> None:
    """From the float32 sums u [T, >= C], C = H*d + G*d + G*vd (q | k | v): every channel through a short causal
    convolution (``conv_w`` float32 [C, taps] or None; the last taps - 1 inputs of every request live at ``state_off``
    of its row of ``state`` and are moved on when ``update_state``); ``norm`` "whole": q and k divided by their root
    mean square over the whole projection times wq [H*d] / wk [G*d], before the rotation; "head": every head divided
    by its own, without weights, after the rotation when ``norm_after``; the first ``rotary_dim`` elements of every
    head of q and k turned by the table rows of ``ctx.positions``; q to q_out [T, H*d], k and v to the token's slot of
    ``kv`` (pages of [G, page_size, d] keys then [G, page_size, vd] values)."""
    T = u.shape[0]
    C = H * d + G * d + G * vd
    assert u.dtype == torch.float32 and u.shape[1] >= C and u.stride(1) == 1
    assert q_out.shape == (T, H * d) and q_out.is_contiguous()
    taps = 0
    if conv_w is not None:
        taps = conv_w.shape[1]
        assert conv_w.shape == (C, taps) and conv_w.dtype == torch.float32 and conv_w.is_contiguous()
        assert taps == 1 or (state is not None and state.dtype == torch.float32 and state.is_contiguous())
    if norm == "whole":
        assert wq.dtype == wk.dtype == torch.float32 and wq.numel() == H * d and wk.numel() == G * d
    if rotary_dim:
        assert cos.dtype == sin.dtype == torch.float32 and cos.shape[1] == rotary_dim // 2
    if write_kv:
        assert kv.numel() % (G * page_size * (d + vd)) == 0 and slot_map.dtype == torch.int32
        _contig(kv, "kv")
    _check(library("qkv_prep").qd_qkv_prep(
        _ptr(u), _LL(u.stride(0)), _I(T), _I(ctx.num_requests), _I(H), _I(G), _I(d), _I(vd), _I(taps), _ptr(conv_w),
        _ptr(state if taps > 1 else None), _LL(state.stride(0) if state is not None else 0), _LL(state_off),
        _ptr(ctx.token_request), _ptr(ctx.cu_tokens), _ptr(ctx.state_slots), _I(1 if update_state else 0),
        _I(QKV_NORMS[norm]), _I(1 if norm_after else 0), _ptr(wq), _ptr(wk), _F(eps), _I(rotary_dim), _I(pairing),
        _ptr(cos), _ptr(sin), _ptr(ctx.positions), _ptr(q_out), _I(dtype_code(q_out.dtype)), _ptr(kv),
        _I(dtype_code(kv.dtype)), _ptr(slot_map), _I(page_size), _I(1 if write_kv else 0), _stream()), "qkv_prep")
    if update_state and taps > 1 and T != ctx.num_requests:
        _launch_count[0] += 1


# ------------------------------------------------------------------ the recurrent mixer with a matrix state
def tm_shift_mix(h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, prev_off: int, ctx, out: torch.Tensor) -> None:
    """out[s, t] = h[t] + (h[t-1] - h[t]) * mu[s]; the row before a portion's first token is the request's kept input
    (``state`` float32 [slots, n], D numbers at ``prev_off``).  h [T, D], mu float32 [n_mix, D], out [n_mix, T, D]."""
    T, D = h.shape
    n = mu.shape[0]
    assert mu.shape == (n, D) and mu.dtype == torch.float32 and out.shape == (n, T, D) and out.dtype == h.dtype
    assert state.dtype == torch.float32
    _contig(h, "h"); _contig(mu, "mu"); _contig(out, "out"); _contig(state, "state")
    _check(library("time_mix").qd_tm_shift_mix(
        _ptr(h), _I(dtype_code(h.dtype)), _I(T), _I(D), _ptr(mu), _I(n), _ptr(state), _LL(state.stride(0)),
        _LL(prev_off), _ptr(ctx.token_request), _ptr(ctx.cu_tokens), _ptr(ctx.state_slots), _ptr(out), _stream()),
        "tm_shift_mix")


def tm_decay(a: torch.Tensor, w2: torch.Tensor, w0: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, c] = exp(-exp(w0[c] + sum_r tanh(a[t, r]) w2[r, c])); a float32 [T, R] (rows may be strided), w2 [R, C]
    (the transpose of the stored matrix), w0 float32 [C], out float32 [T, C]."""
    T, R = a.shape
    C = w2.shape[1]
    assert a.dtype == torch.float32 and a.stride(1) == 1 and w2.shape == (R, C) and w0.dtype == torch.float32
    assert w0.numel() == C and out.shape == (T, C) and out.dtype == torch.float32
    _contig(w2, "w2"); _contig(out, "out")
    _check(library("time_mix").qd_tm_decay(_ptr(a), _LL(a.stride(0)), _I(T), _I(R), _ptr(w2), _I(dtype_code(w2.dtype)),
                                           _ptr(w0), _I(C), _ptr(out), _stream()), "tm_decay")


def tm_scan(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, u: torch.Tensor, H: int, d: int,
            state: torch.Tensor, s_off: int, ctx, out: torch.Tensor, write_state: bool) -> None:
    """Per (request, head), token by token: o_t = (S + diag(u) k_t v_t^T)^T r_t; S <- diag(w_t) S + k_t v_t^T.
    r, k, v float32 [T, H*d] with one common row stride (column ranges of one tensor), w float32 [T, H*d] dense,
    u float32 [H, d], out float32 [T, H*d]; S [H, d, d] at ``s_off`` of the request's row of ``state``."""
    T = r.shape[0]
    assert r.dtype == k.dtype == v.dtype == w.dtype == out.dtype == torch.float32
    assert r.shape == k.shape == v.shape == w.shape == out.shape == (T, H * d)
    assert r.stride(0) == k.stride(0) == v.stride(0) and r.stride(1) == k.stride(1) == v.stride(1) == 1
    assert u.shape == (H, d) and u.dtype == torch.float32 and state.dtype == torch.float32
    _contig(w, "w"); _contig(out, "out"); _contig(u, "u"); _contig(state, "state")
    _check(library("time_mix").qd_tm_scan(
        _ptr(r), _ptr(k), _ptr(v), _LL(r.stride(0)), _ptr(w), _ptr(u), _I(H), _I(d), _I(d), _ptr(state),
        _LL(state.stride(0)), _LL(s_off), _ptr(ctx.cu_tokens), _ptr(ctx.state_slots), _I(ctx.num_requests), _ptr(out),
        _I(1 if write_state else 0), _stream()), "tm_scan")


def tm_finish(o: torch.Tensor, g: torch.Tensor, norm: torch.Tensor, H: int, d: int, eps: float, out_scale: float,
              out: torch.Tensor, h: torch.Tensor, state: torch.Tensor, prev_off: int, ctx, write_state: bool) -> None:
    """out[t, head] = o / sqrt(mean(o^2) + eps) * norm * silu(g) * out_scale per head of d values; o float32
    [T, H*d], g float32 [T, H*d] (rows may be strided), norm float32 [H*d]; out [T, H*d] (rows may be strided).  The
    last token of every portion leaves its row of h [T, D] as the request's kept input at ``prev_off``."""
    T = o.shape[0]
    assert o.dtype == g.dtype == norm.dtype == torch.float32 and o.shape == g.shape == out.shape == (T, H * d)
    assert g.stride(1) == 1 and out.stride(1) == 1 and norm.numel() == H * d
    _contig(o, "o"); _contig(h, "h"); _contig(state, "state")
    _check(library("time_mix").qd_tm_finish(
        _ptr(o), _ptr(g), _LL(g.stride(0)), _ptr(norm), _I(T), _I(H), _I(d), _F(eps), _F(out_scale), _ptr(out),
        _I(dtype_code(out.dtype)), _LL(out.stride(0)), _ptr(h), _I(dtype_code(h.dtype)), _I(h.shape[1]), _ptr(state),
        _LL(state.stride(0)), _LL(prev_off), _ptr(ctx.token_request), _ptr(ctx.cu_tokens), _ptr(ctx.state_slots),
        _I(1 if write_state else 0), _stream()), "tm_finish")


# ------------------------------------------------------------------ the layers of a prompt step from native code
class PromptLayer(ctypes.Structure):
    """One schedule entry of the native prompt step (PeLayer in csrc/prompt_exec.cu)."""
    _fields_ = [(n, ctypes.c_void_p) for n in ("norm1_w", "norm2_w", "wqkv", "bqkv", "wo", "wgu", "wd", "kv")] + \
        [("eps1", ctypes.c_float), ("eps2", ctypes.c_float), ("write_kv", ctypes.c_int), ("pad", ctypes.c_int)]


class PromptFns(ctypes.Structure):
    """Addresses of the launchers and of the library product that the native prompt step calls."""
    _fields_ = [(n, ctypes.c_void_p) for n in ("add_rmsnorm", "rope_kv_write", "swiglu", "attention_regs",
                                               "attention_tc5", "attention_decode", "gemm_ex", "blas",
                                               "gemm_batched", "plain_next")]


class PromptParams(ctypes.Structure):
    """Arguments of the native prompt step (PeParams in csrc/prompt_exec.cu)."""
    _fields_ = [("fn", PromptFns), ("layers", ctypes.c_void_p), ("n_layers", ctypes.c_int)] + \
        [(n, ctypes.c_int) for n in ("T", "R", "D", "H", "G", "d", "F", "page_size", "window", "rotary_dim",
                                     "pairing", "max_blocks", "use_tc5", "n_wanted")] + \
        [("scale", ctypes.c_float), ("final_eps", ctypes.c_float), ("n_pages", ctypes.c_longlong)] + \
        [(n, ctypes.c_void_p) for n in ("positions", "slot_map", "block_table", "cu_tokens", "start_pos",
                                        "logit_rows", "cos_t", "sin_t", "final_w", "x", "delta0", "h", "qkv",
                                        "attn", "delta", "gu", "act", "hrows")] + \
        [("n_decode", ctypes.c_int), ("decode_splits", ctypes.c_int)] + \
        [(n, ctypes.c_void_p) for n in ("token_req", "part_o", "part_ml", "tickets", "down_part")] + \
        [("down_shares", ctypes.c_int), ("pad2", ctypes.c_int)]


def prompt_exec_struct_sizes_match() -> bool:
    a, b = ctypes.c_int(0), ctypes.c_int(0)
    library("prompt_exec").qd_prompt_exec_struct_sizes(ctypes.byref(a), ctypes.byref(b))
    return a.value == ctypes.sizeof(PromptLayer) and b.value == ctypes.sizeof(PromptParams)


def _loaded_cublas() -> ctypes.CDLL:
    """The cuBLAS that this process has loaded already (torch's), found among the mapped files: the native
    prompt step must call the same copy whose handle it is given."""
    torch.cuda.current_blas_handle()          # makes torch load and initialise it
    with open("/proc/self/maps") as f:
        for line in f:
            path = line.split(None, 5)[-1].strip() if line.count("/") else ""
            if "/libcublas.so" in path:
                return ctypes.CDLL(path)
    raise KernelError("no libcublas is loaded in this process")


_prompt_fns: dict = {}


def prompt_fns(use_tc5: bool, with_decode: bool = False) -> PromptFns:
    """The launchers' addresses (their libraries are built and loaded on the first call; an attention
    kernel that the model does not use stays unbuilt); ``blas`` is filled in per step."""
    fns = _prompt_fns.get((use_tc5, with_decode))
    if fns is None:
        addr = lambda f: ctypes.cast(f, ctypes.c_void_p).value
        ew = library("elementwise")
        fns = PromptFns()
        fns.add_rmsnorm = addr(ew.qd_add_rmsnorm)
        fns.rope_kv_write = addr(ew.qd_rope_kv_write_biased)
        fns.swiglu = addr(ew.qd_swiglu)
        if use_tc5:
            fns.attention_tc5 = addr(library("attention_tc5").qd_prefill_attention_tc5)
        else:
            fns.attention_regs = addr(library("attention_flash").qd_prefill_attention)
        if with_decode:
            fns.attention_decode = addr(library("attention_flash").qd_decode_attention)
        fns.gemm_ex = addr(_loaded_cublas().cublasGemmEx)
        fns.gemm_batched = addr(_loaded_cublas().cublasGemmStridedBatchedEx)
        fns.plain_next = addr(ew.qd_elementwise_plain_next)
        _prompt_fns[(use_tc5, with_decode)] = fns
    return fns


def decode_scratch(n_tokens: int, H: int, d: int, G: int, splits: int, device):
    """(part_o, part_ml, tickets) for a split-KV decode attention launch of ``n_tokens`` tokens."""
    if splits <= 1:
        return None, None, None
    part_o = torch.empty((n_tokens * H * splits, d), dtype=torch.float32, device=device)
    part_ml = torch.empty((n_tokens * H * splits, 2), dtype=torch.float32, device=device)
    tickets = None
    if n_tokens * G <= _TICKETS:
        tickets = _tickets.get(device)
        if tickets is None:     # zero once; every launch leaves them zero again
            tickets = _tickets[device] = torch.zeros(_TICKETS, dtype=torch.int32, device=device)
    return part_o, part_ml, tickets


def prompt_exec(params: PromptParams, n_launches: int) -> None:
    """All layers of a prompt step and the final norm at the wanted rows, launched from one native loop on
    the step's stream (``params.fn.blas`` must be a cuBLAS handle bound to that stream)."""
    stream = _stream()
    _launch_count[0] += n_launches - 1
    code = library("prompt_exec").qd_prompt_exec(ctypes.byref(params), stream)
    if code >= 20000:
        raise KernelError(f"prompt_exec: cuBLAS status {code - 20000}")
    _check(code, "prompt_exec")
