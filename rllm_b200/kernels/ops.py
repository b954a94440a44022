"""Python faces of the CUDA kernels: torch tensors in, kernel launched on the
current stream.  There is no fallback: a tensor that is not on a CUDA device,
a missing compiler or a size that a kernel refuses raises an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build

DT_F32, DT_BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt is torch.float32:
        return DT_F32
    if dt is torch.bfloat16:
        return DT_BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dt}")


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("the engine's kernels run on CUDA tensors only; there is no CPU path")
    return c_void_p(t.data_ptr())


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


LAUNCHES = [0]      # entry-point calls so far (each launches at least one kernel)


def _check(code: int, what: str) -> None:
    LAUNCHES[0] += 1
    if code == 0:
        return
    if code == -1:
        raise KernelError(f"{what}: refused its arguments (bad size or pointer)")
    if code == -2:
        raise KernelError(f"{what}: this size is legal but no kernel of this build takes it")
    raise KernelError(f"{what}: CUDA error {code}")


def _contig(t: torch.Tensor, name: str) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


# ---------------------------------------------------------------------------
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: torch.Tensor,
              scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] * scale as float32; ids int32 [T], out float32 [T, H], or [C, T, H]: C copies."""
    lib = build.load_library("elementwise")
    T, (V, H) = ids.numel(), table.shape
    copies = out.shape[0] if out.dim() == 3 else 1
    assert ids.dtype is torch.int32 and out.dtype is torch.float32 and out.shape[-2:] == (T, H)
    _contig(table, "table"); _contig(out, "out")
    _check(lib.rllm_embedding(_ptr(ids), _ptr(table), c_int(dtype_code(table.dtype)), _ptr(out),
                              c_int(T), c_int(H), c_int(V), c_float(scale), c_int(copies), _ptr(err), _stream()),
           "embedding")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
            writeback: bool = False) -> None:
    """out = rmsnorm(x [+ delta]) * weight; x float32 [., H]; out [R, H] in the
    activation dtype.  ``writeback`` stores x + delta into x.  ``rows`` (int32
    [R]) picks the input row of each output row."""
    lib = build.load_library("elementwise")
    H = x.shape[-1]
    R = out.shape[0]
    assert x.dtype is torch.float32 and out.shape[-1] == H and weight.numel() == H
    _contig(x, "x"); _contig(out, "out"); _contig(weight, "weight")
    if delta is not None:
        assert delta.dtype is out.dtype and delta.shape == x.shape
        _contig(delta, "delta")
    if rows is not None:
        assert rows.dtype is torch.int32 and rows.numel() == R
    else:
        assert x.shape[0] == R
    _check(lib.rllm_rmsnorm(_ptr(x), _ptr(delta), _ptr(rows), _ptr(weight),
                            c_int(dtype_code(weight.dtype)), _ptr(out), c_int(dtype_code(out.dtype)),
                            c_int(R), c_int(H), c_float(eps), c_int(1 if writeback else 0), _stream()),
           "rmsnorm")


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> None:
    lib = build.load_library("elementwise")
    assert x.dtype is torch.float32 and x.shape == delta.shape
    _contig(x, "x"); _contig(delta, "delta")
    _check(lib.rllm_residual_add(_ptr(x), _ptr(delta), c_int(dtype_code(delta.dtype)),
                                 c_longlong(x.numel()), _stream()), "residual_add")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor,
                  inv_freq: Optional[torch.Tensor], rotary_dim: int, block_table: Optional[torch.Tensor],
                  kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor], nq: int, nkv: int,
                  d: int, err: torch.Tensor, write_kv: bool = True) -> None:
    """Rotates q (in place) and k, stores k and v of every token into its page.

    qkv [T, (nq + 2 nkv) d]; caches [pages, nkv, page_size, d]; inv_freq float64
    [rotary_dim / 2]; block_table int32 [S, max_blocks]."""
    lib = build.load_library("elementwise")
    T = qkv.shape[0]
    assert qkv.shape[1] == (nq + 2 * nkv) * d
    _contig(qkv, "qkv")
    if rotary_dim:
        assert inv_freq is not None and inv_freq.dtype is torch.float64 and inv_freq.numel() == rotary_dim // 2
    if write_kv:
        assert kcache.dtype is qkv.dtype and vcache.dtype is qkv.dtype
        assert kcache.shape == vcache.shape and kcache.shape[1] == nkv and kcache.shape[3] == d
        _contig(kcache, "kcache"); _contig(vcache, "vcache"); _contig(block_table, "block_table")
        pages, page_size, max_blocks = kcache.shape[0], kcache.shape[2], block_table.shape[1]
    else:
        pages = page_size = max_blocks = 0
    _check(lib.rllm_rope_kv_write(_ptr(qkv), c_int(dtype_code(qkv.dtype)), _ptr(positions),
                                  _ptr(token_seq), _ptr(inv_freq), c_int(rotary_dim),
                                  _ptr(block_table), c_int(max_blocks), _ptr(kcache), _ptr(vcache),
                                  c_int(T), c_int(nq), c_int(nkv), c_int(d), c_int(page_size),
                                  c_int(pages), c_int(1 if write_kv else 0), _ptr(err), _stream()),
           "rope_kv_write")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    lib = build.load_library("elementwise")
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and gate_up.dtype is out.dtype
    _contig(gate_up, "gate_up"); _contig(out, "out")
    _check(lib.rllm_silu_mul(_ptr(gate_up), _ptr(out), c_int(dtype_code(out.dtype)), c_int(T), c_int(I),
                             _stream()), "silu_mul")


def attention_simt(q: torch.Tensor, q_stride: int, out: torch.Tensor, kcache: torch.Tensor,
                   vcache: torch.Tensor, block_table: torch.Tensor, positions: torch.Tensor,
                   token_seq: torch.Tensor, nq: int, nkv: int, d: int, window: int, scale: float,
                   err: torch.Tensor) -> None:
    """Paged causal attention of T query tokens, one warp per (token, head).

    q: T rows of nq*d values with row stride q_stride (elements); out [T, nq*d]."""
    lib = build.load_library("attention_simt")
    T = out.shape[0]
    _contig(out, "out"); _contig(kcache, "kcache"); _contig(vcache, "vcache"); _contig(block_table, "block_table")
    assert kcache.dtype is q.dtype and out.dtype is q.dtype
    _check(lib.rllm_attention_simt(_ptr(q), c_int(q_stride), _ptr(out), _ptr(kcache), _ptr(vcache),
                                   c_int(dtype_code(q.dtype)), _ptr(block_table),
                                   c_int(block_table.shape[1]), _ptr(positions), _ptr(token_seq),
                                   c_int(T), c_int(nq), c_int(nkv), c_int(d), c_int(kcache.shape[2]),
                                   c_int(kcache.shape[0]), c_int(window), c_float(scale), _ptr(err),
                                   _stream()), "attention_simt")


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] . w[N, K]^T, float32 FFMA."""
    lib = build.load_library("gemm_f32")
    M, K = a.shape
    N = w.shape[0]
    assert a.dtype is torch.float32 and w.dtype is torch.float32 and out.dtype is torch.float32
    assert w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(lib.rllm_gemm_f32(_ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out),
                             c_int(out.stride(0)), c_int(M), c_int(N), c_int(K), _stream()), "gemm_f32")


SMALL_M_MAX = 8       # up to here the weight-streaming GEMM beats the library's on a B200 (it takes 16)
FUSED_M_MAX = 16      # up to here a step goes through the forms of it that carry the residual add and the norm
                      # (RLLM_FUSED_M_MAX in the environment overrides it, for measurements).  Measured at
                      # context 4096: batch 12 1.32 -> 1.06 ms a step, batch 16 1.39 -> 1.16 ms, against the
                      # library's products with norm and SiLU kernels between them


def gemm_small_m(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: str = "store") -> None:
    """out = x . w^T for M <= 16 rows of bfloat16, bound by one read of w.
    epilogue "store": out [M, N] bfloat16 or float32.  "silu_mul": w = [gate rows;
    up rows] stacked (2 N rows), out [M, N] bfloat16 = silu(x gate^T) * (x up^T)."""
    lib = build.load_library("gemm_small_m")
    M, K = x.shape
    assert x.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and w.shape[1] == K
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if epilogue == "silu_mul":
        N = w.shape[0] // 2
        assert out.dtype is torch.bfloat16 and out.shape == (M, N) and w.shape[0] == 2 * N
        code = 2
    else:
        N = w.shape[0]
        assert out.shape == (M, N)
        code = 1 if out.dtype is torch.float32 else 0
        assert out.dtype in (torch.float32, torch.bfloat16)
    _check(lib.rllm_gemm_small_m(_ptr(x), c_int(x.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out),
                                 c_int(out.stride(0)), c_int(M), c_int(N), c_int(K), c_int(code), _stream()),
           "gemm_small_m")


def gemm_small_m_residual(x: torch.Tensor, w: torch.Tensor, h: torch.Tensor,
                          w_next: Optional[torch.Tensor]):
    """h += x . w^T (h float32, in place) for M <= 16 rows of bfloat16.  Returns
    (parts, scaled): parts float32 [P, M], whose sum over P is each row's new sum of
    squares; scaled = bfloat16(h * w_next) [M, N] if the weight ``w_next`` of the norm
    that reads h next is given, else None."""
    lib = build.load_library("gemm_small_m")
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and w.shape[1] == K
    assert h.dtype is torch.float32 and h.shape == (M, N) and h.stride(1) == 1
    assert x.stride(1) == 1 and w.stride(1) == 1
    P = int(lib.rllm_gemm_small_m_parts(c_int(N)))
    parts = torch.empty((P, M), dtype=torch.float32, device=x.device)
    scaled = None
    if w_next is not None:
        assert w_next.numel() == N and w_next.is_contiguous() and w_next.dtype in (torch.float32, torch.bfloat16)
        scaled = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    _check(lib.rllm_gemm_small_m_residual(_ptr(x), c_int(x.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(h),
                                          c_int(h.stride(0)), _ptr(parts), _ptr(w_next),
                                          c_int(1 if w_next is not None and w_next.dtype is torch.float32 else 0),
                                          _ptr(scaled), c_int(N), c_int(M), c_int(N), c_int(K), _stream()),
           "gemm_small_m_residual")
    return parts, scaled


def gemm_small_m_rstd(x: torch.Tensor, parts: torch.Tensor, eps: float, w: torch.Tensor, out: torch.Tensor,
                      epilogue: str = "store") -> None:
    """out = (x . w^T) with row m scaled by 1 / sqrt(sum(parts[:, m]) / K + eps): with
    x and parts from ``gemm_small_m_residual`` this is rmsnorm(h) . w^T.  Epilogues
    as in ``gemm_small_m`` (bfloat16 out)."""
    lib = build.load_library("gemm_small_m")
    M, K = x.shape
    assert x.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and w.shape[1] == K and out.dtype is torch.bfloat16
    assert parts.dtype is torch.float32 and parts.is_contiguous() and parts.shape[1] == M
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if epilogue == "silu_mul":
        N, code = w.shape[0] // 2, 2
        assert w.shape[0] == 2 * N
    else:
        N, code = w.shape[0], 0
    assert out.shape == (M, N)
    _check(lib.rllm_gemm_small_m_rstd(_ptr(x), c_int(x.stride(0)), _ptr(parts), c_int(parts.shape[0]), c_float(eps),
                                      _ptr(w), c_int(w.stride(0)), _ptr(out), c_int(out.stride(0)), c_int(M),
                                      c_int(N), c_int(K), c_int(code), _stream()), "gemm_small_m_rstd")


_one_wave_tiles = {}


def small_m_rows(num_rows: int, dtype: torch.dtype, weights=()) -> bool:
    """Whether a step of this many rows goes through the weight-streaming kernels.  Up to 8 rows: always.
    9 to 16 rows: if every one of ``weights`` has few enough rows for the kernels' one-wave form (16 rows a
    CTA, seven CTAs an SM); measured at batch 16, context 4096, four layers: Llama-1B shapes 16 % faster
    than the library path, 3B shapes equal, 8B shapes (whose gate_up has too many rows) 6 % slower."""
    import os
    if dtype is not torch.bfloat16 or num_rows <= 0 or os.environ.get("RLLM_GEMM") == "library":
        return False
    if num_rows > int(os.environ.get("RLLM_FUSED_M_MAX", FUSED_M_MAX)):
        return False
    if num_rows <= SMALL_M_MAX:
        return True
    for w in weights:
        cap = _one_wave_tiles.get(w.device)
        if cap is None:
            cap = _one_wave_tiles[w.device] = 7 * torch.cuda.get_device_properties(w.device).multi_processor_count
        if w.shape[0] // 16 > cap:
            return False
    return True


def small_m_takes(x: torch.Tensor, w: torch.Tensor) -> bool:
    import os
    return (x.dtype is torch.bfloat16 and 0 < x.shape[0] <= SMALL_M_MAX and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and os.environ.get("RLLM_GEMM") != "library")


_gemm_err = {}


def gemm_error_word(device: torch.device) -> torch.Tensor:
    """The per-device error word of the tcgen05 GEMM (bit 4: a bounded wait ran out)."""
    t = _gemm_err.get(device)
    if t is None:
        t = _gemm_err[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return t


def check_gemm_errors(device: torch.device) -> None:
    t = _gemm_err.get(device)
    code = int(t.item()) if t is not None else 0
    if code:
        t.zero_()
        what = []
        if code & 16:
            what.append("gemm_tcgen05: a wait on an mbarrier ran out")
        raise KernelError("; ".join(what or [f"error word {code}"]) + "; the result of that product is undefined")


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: str = "store") -> None:
    """out = x . w^T for bfloat16 on the tcgen05 tensor cores (TMA in, TMEM accumulators).
    epilogue "store": out [M, N] bfloat16 or float32.  "silu_mul": w = [gate rows;
    up rows] stacked (2 N rows), out [M, N] bfloat16 = silu(x gate^T) * (x up^T)."""
    lib = build.load_library("gemm_tcgen05")
    M, K = x.shape
    assert x.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and w.shape[1] == K
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if epilogue == "silu_mul":
        N = w.shape[0] // 2
        assert out.dtype is torch.bfloat16 and out.shape == (M, N) and w.shape[0] == 2 * N
        code = 2
    else:
        N = w.shape[0]
        assert out.shape == (M, N) and out.dtype in (torch.float32, torch.bfloat16)
        code = 1 if out.dtype is torch.float32 else 0
    _check(lib.rllm_gemm_tcgen05(_ptr(x), c_int(x.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out),
                                 c_int(out.stride(0)), c_int(M), c_int(N), c_int(K), c_int(code),
                                 _ptr(gemm_error_word(x.device)), _stream()), "gemm_tcgen05")


TCGEN05_MIN_TILES = 96    # below this many 128 x 256 output tiles the GPU is not filled: the library's
                          # small-tile kernels read the weight faster


def tcgen05_takes(x: torch.Tensor, w: torch.Tensor, silu: bool = False) -> bool:
    """Whether the tcgen05 kernel should compute x . w^T.  ``silu``: w is [gate; up] stacked and the
    output has half of w's rows.  With the environment variable RLLM_GEMM=tcgen05 every shape it can
    take goes to it (used by tests, so that tiny models run through it)."""
    import os
    mode = os.environ.get("RLLM_GEMM", "")
    if mode in ("library", "no_tcgen05"):
        return False
    ok = (x.dtype is torch.bfloat16 and x.shape[0] > 0 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
          and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)
    if not ok or mode == "tcgen05":
        return ok
    n_out = w.shape[0] // 2 if silu else w.shape[0]
    tiles = -(-x.shape[0] // 128) * -(-n_out // (128 if silu else 256))
    return tiles >= TCGEN05_MIN_TILES


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> Optional[torch.Tensor]:
    """x . w^T through this engine's own bfloat16 kernels, or None if none of them
    takes the shape (the caller then uses the library's matrix product).  Few rows:
    the weight-streaming kernel; more: the tcgen05 kernel."""
    if small_m_takes(x, w):
        import os
        if w.shape[0] > 65536 and (x.shape[0] > 8 or os.environ.get("RLLM_HEAD") == "library"):
            return None                 # very tall weights (the vocabulary) at 9 to 16 rows: the library's kernel is ahead
        out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
        gemm_small_m(x, w, out)
        return out
    if tcgen05_takes(x, w):
        out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
        gemm_tcgen05(x, w, out)
        return out
    return None


# ---------------------------------------------------------------------------
def draw_normal(out: torch.Tensor, key: int, std: float, one_plus: bool = False) -> None:
    """Fills ``out`` (float32 or bfloat16, contiguous) with std * z or 1 + std * z, z the standard normals
    of the counter-based stream ``key``: element i is the same value wherever it is drawn
    (``rllm_b200.weights.counter_rng`` is the CPU twin)."""
    lib = build.load_library("weights_rng")
    _contig(out, "out")
    _check(lib.rllm_draw_normal(_ptr(out), c_int(dtype_code(out.dtype)), c_longlong(out.numel()),
                                ctypes.c_ulonglong(key & 0xFFFFFFFFFFFFFFFF), ctypes.c_double(std),
                                c_int(1 if one_plus else 0), _stream()), "draw_normal")


def draw_randint(out: torch.Tensor, key: int, high: int) -> None:
    """Fills ``out`` (int32, contiguous) with word i of the stream ``key`` modulo ``high``."""
    lib = build.load_library("weights_rng")
    assert out.dtype is torch.int32 and 0 < high < (1 << 32)
    _contig(out, "out")
    _check(lib.rllm_draw_randint(_ptr(out), c_longlong(out.numel()), ctypes.c_ulonglong(key & 0xFFFFFFFFFFFFFFFF),
                                 ctypes.c_uint(high), _stream()), "draw_randint")


# ---------------------------------------------------------------------------
_argmax_scratch = {}


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = lowest index of the largest value of row r (float32 rows)."""
    lib = build.load_library("sampling")
    R, V = logits.shape
    assert logits.dtype is torch.float32 and out.dtype is torch.int32 and logits.stride(1) == 1
    split = int(lib.rllm_argmax_split(c_int(V)))
    scratch = _argmax_scratch.get(logits.device)
    if scratch is None or scratch[1].numel() < R:
        rows = max(R, 256)
        scratch = (torch.empty(rows * 64 * 2, dtype=torch.int32, device=logits.device),
                   torch.zeros(rows, dtype=torch.int32, device=logits.device))
        _argmax_scratch[logits.device] = scratch
    _check(lib.rllm_argmax(_ptr(logits), c_int(R), c_int(V), c_int(logits.stride(0)), _ptr(out),
                           _ptr(scratch[0]), _ptr(scratch[1]), _stream()), "argmax")


def _sample_asserts(logits, temperature, top_k, top_p, min_p, seeds, gen_index, out):
    assert logits.dtype is torch.float32 and logits.stride(1) == 1
    assert temperature.dtype is torch.float32 and top_k.dtype is torch.int32
    assert top_p.dtype is torch.float32 and min_p.dtype is torch.float32
    assert seeds.dtype is torch.int64 and gen_index.dtype is torch.int64 and out.dtype is torch.int32


_sample_scratch = {}


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, seeds: torch.Tensor, gen_index: torch.Tensor, out: torch.Tensor,
           with_select: bool = True) -> None:
    """out[r] = the next token of row r: argmax for greedy rows, else a draw after temperature, top-k,
    top-p and min-p.  Every row is worked on by several CTAs, in a chain of small kernels.
    ``with_select=False`` leaves the top-k / top-p kernels out (the caller knows that no row uses them)."""
    lib = build.load_library("sampling")
    R, V = logits.shape
    _sample_asserts(logits, temperature, top_k, top_p, min_p, seeds, gen_index, out)
    lib.rllm_sample_scratch_bytes.restype = c_longlong
    need = int(lib.rllm_sample_scratch_bytes(c_int(R), c_int(V)))
    scratch = _sample_scratch.get(logits.device)
    if scratch is None or scratch.numel() < need:
        scratch = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=logits.device)
        _sample_scratch[logits.device] = scratch
    _check(lib.rllm_sample(_ptr(logits), c_int(R), c_int(V), c_int(logits.stride(0)), _ptr(temperature),
                           _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(seeds), _ptr(gen_index), _ptr(out),
                           _ptr(scratch), c_int(1 if with_select else 0), _stream()), "sample")


def sample_one_cta(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                   min_p: torch.Tensor, seeds: torch.Tensor, gen_index: torch.Tensor, out: torch.Tensor) -> None:
    """The same sampling with one CTA a row in one kernel (slow for large vocabularies; kept as the
    simple form that the chain of kernels is checked against)."""
    lib = build.load_library("sampling")
    R, V = logits.shape
    _sample_asserts(logits, temperature, top_k, top_p, min_p, seeds, gen_index, out)
    _check(lib.rllm_sample_one_cta(_ptr(logits), c_int(R), c_int(V), c_int(logits.stride(0)), _ptr(temperature),
                                   _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(seeds), _ptr(gen_index),
                                   _ptr(out), _stream()), "sample_one_cta")


def logit_edits(logits: torch.Tensor, rows: torch.Tensor, tokens: torch.Tensor, counts: torch.Tensor,
                bias: torch.Tensor, rep: torch.Tensor, freq: torch.Tensor, pres: torch.Tensor) -> None:
    lib = build.load_library("sampling")
    R, V = logits.shape
    _check(lib.rllm_logit_edits(_ptr(logits), c_int(V), c_int(logits.stride(0)), c_int(rows.numel()),
                                _ptr(rows), _ptr(tokens), _ptr(counts), _ptr(bias), _ptr(rep),
                                _ptr(freq), _ptr(pres), _stream()), "logit_edits")


def logit_mask(logits: torch.Tensor, allowed_start: Optional[torch.Tensor],
               allowed: Optional[torch.Tensor], sup_rows: Optional[torch.Tensor],
               sup_tokens: Optional[torch.Tensor]) -> None:
    lib = build.load_library("sampling")
    R, V = logits.shape
    n = 0 if sup_rows is None else sup_rows.numel()
    _check(lib.rllm_logit_mask(_ptr(logits), c_int(R), c_int(V), c_int(logits.stride(0)),
                               _ptr(allowed_start), _ptr(allowed), c_int(n), _ptr(sup_rows),
                               _ptr(sup_tokens), _stream()), "logit_mask")


def attention_prefill_bf16(q: torch.Tensor, q_stride: int, out: torch.Tensor, kcache: torch.Tensor,
                           vcache: torch.Tensor, block_table: torch.Tensor, q_start: torch.Tensor,
                           seq_lens: torch.Tensor, seq_begin: int, seq_end: int, num_tokens: int, nq: int,
                           nkv: int, d: int, window: int, scale: float, err: torch.Tensor, keep_first: int = 0,
                           chunk: int = 0, softcap: float = 0.0, sinks: Optional[torch.Tensor] = None,
                           gate: Optional[torch.Tensor] = None, gate_per_head: bool = False,
                           slopes: Optional[torch.Tensor] = None) -> None:
    """Tensor-core attention of the prompt portions of sequences seq_begin .. seq_end-1.  ``keep_first``,
    ``chunk``, ``softcap``, ``sinks``, ``gate`` and ``slopes`` as in ``attention_simt_kv`` (gate: a row per row of q)."""
    lib = build.load_library("attention_mma")
    _contig(out, "out"); _contig(kcache, "kcache"); _contig(vcache, "vcache"); _contig(block_table, "block_table")
    assert q.dtype is torch.bfloat16 and kcache.dtype is torch.bfloat16 and out.dtype is torch.bfloat16
    if keep_first or chunk or softcap or sinks is not None or gate is not None or slopes is not None:
        gate_mode = _attention_opts_asserts(sinks, gate, gate_per_head, nq, d, slopes)
        _check(lib.rllm_attention_prefill_bf16_opts(
            _ptr(q), c_int(q_stride), _ptr(out), _ptr(kcache), _ptr(vcache), _ptr(block_table),
            c_int(block_table.shape[1]), _ptr(q_start), _ptr(seq_lens), c_int(seq_begin), c_int(seq_end),
            c_int(num_tokens), c_int(nq), c_int(nkv), c_int(d), c_int(kcache.shape[2]), c_int(kcache.shape[0]),
            c_int(window), c_float(scale), c_int(keep_first), c_int(chunk), c_float(softcap), _ptr(sinks), _ptr(gate),
            c_int(gate.stride(0) if gate is not None else 0), c_int(gate_mode), _ptr(slopes), _ptr(err), _stream()),
            "attention_prefill_bf16_opts")
        return
    _check(lib.rllm_attention_prefill_bf16(_ptr(q), c_int(q_stride), _ptr(out), _ptr(kcache), _ptr(vcache),
                                           _ptr(block_table), c_int(block_table.shape[1]), _ptr(q_start),
                                           _ptr(seq_lens), c_int(seq_begin), c_int(seq_end), c_int(num_tokens),
                                           c_int(nq), c_int(nkv), c_int(d), c_int(kcache.shape[2]),
                                           c_int(kcache.shape[0]), c_int(window), c_float(scale), _ptr(err),
                                           _stream()), "attention_prefill_bf16")


def attention_prefill_tcgen05_supported(nq: int, nkv: int, d: int, page_size: int) -> bool:
    """The sizes the tcgen05 prompt attention takes: head size 64 or 128, pages of 16 keys up to a key
    tile (128 keys for head size 64, 64 for 128), up to 128 query heads per kv head."""
    g = nq // nkv if nkv else 0
    return (d in (64, 128) and page_size in (16, 32, 64, 128) and page_size <= 8192 // d
            and 1 <= g <= 128 and nq % nkv == 0)


def attention_prefill_tcgen05(q: torch.Tensor, q_stride: int, out: torch.Tensor, kcache: torch.Tensor,
                              vcache: torch.Tensor, block_table: torch.Tensor, q_start: torch.Tensor,
                              seq_lens: torch.Tensor, seq_begin: int, seq_end: int, num_tokens: int, nq: int,
                              nkv: int, d: int, window: int, scale: float, err: torch.Tensor, keep_first: int = 0,
                              chunk: int = 0, softcap: float = 0.0, sinks: Optional[torch.Tensor] = None,
                              gate: Optional[torch.Tensor] = None, gate_per_head: bool = False,
                              slopes: Optional[torch.Tensor] = None) -> None:
    """Attention of the prompt portions of sequences seq_begin .. seq_end-1 on the
    tcgen05 tensor cores (same contract and options as ``attention_prefill_bf16``; ``q`` is the
    first of ``q.shape[0]`` rows of ``q_stride`` elements)."""
    lib = build.load_library("attention_tcgen05")
    _contig(out, "out"); _contig(kcache, "kcache"); _contig(vcache, "vcache"); _contig(block_table, "block_table")
    assert q.dtype is torch.bfloat16 and kcache.dtype is torch.bfloat16 and out.dtype is torch.bfloat16
    if keep_first or chunk or softcap or sinks is not None or gate is not None or slopes is not None:
        gate_mode = _attention_opts_asserts(sinks, gate, gate_per_head, nq, d, slopes)
        _check(lib.rllm_attention_prefill_tcgen05_opts(
            _ptr(q), c_int(q_stride), c_int(q.shape[0]), _ptr(out), _ptr(kcache), _ptr(vcache), _ptr(block_table),
            c_int(block_table.shape[1]), _ptr(q_start), _ptr(seq_lens), c_int(seq_begin), c_int(seq_end),
            c_int(num_tokens), c_int(nq), c_int(nkv), c_int(d), c_int(kcache.shape[2]), c_int(kcache.shape[0]),
            c_int(window), c_float(scale), c_int(keep_first), c_int(chunk), c_float(softcap), _ptr(sinks), _ptr(gate),
            c_int(gate.stride(0) if gate is not None else 0), c_int(gate_mode), _ptr(slopes), _ptr(err), _stream()),
            "attention_prefill_tcgen05_opts")
        return
    _check(lib.rllm_attention_prefill_tcgen05(_ptr(q), c_int(q_stride), c_int(q.shape[0]), _ptr(out), _ptr(kcache),
                                              _ptr(vcache), _ptr(block_table), c_int(block_table.shape[1]),
                                              _ptr(q_start), _ptr(seq_lens), c_int(seq_begin), c_int(seq_end),
                                              c_int(num_tokens), c_int(nq), c_int(nkv), c_int(d),
                                              c_int(kcache.shape[2]), c_int(kcache.shape[0]), c_int(window),
                                              c_float(scale), _ptr(err), _stream()), "attention_prefill_tcgen05")


_decode_counters = {}
_retired_counters = []          # buffers that grew out of use: captured graphs may still hold their address


def _attention_opts_asserts(sinks, gate, gate_per_head: bool, nq: int, d: int, slopes=None) -> int:
    """Checks of the tensor-core kernels' options; returns the kernels' gate mode."""
    if slopes is not None:
        assert slopes.dtype is torch.float32 and slopes.numel() == nq and slopes.is_contiguous()
    if sinks is not None:
        assert sinks.dtype is torch.float32 and sinks.numel() == nq and sinks.is_contiguous()
    if gate is None:
        return 0
    assert gate.dtype is torch.bfloat16 and gate.stride(1) == 1 and gate.shape[1] == (nq if gate_per_head else nq * d)
    return 1 if gate_per_head else 2


def _counters_for(device: torch.device, n: int) -> torch.Tensor:
    """Zeroed per-device counters of the decode kernel's split merge; the kernel
    leaves them zero, so one buffer serves every call (also under CUDA graphs).
    A buffer that is outgrown is never freed (a captured graph replays with its
    address), and none is made while a stream is being captured."""
    buf = _decode_counters.get(device)
    if buf is None or buf.numel() < n:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError(f"attention_decode: {n} merge counters are needed and the buffer cannot grow during "
                              "a stream capture; run this size once outside a capture first")
        if buf is not None:
            _retired_counters.append(buf)
        buf = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)
        _decode_counters[device] = buf
    return buf


def attention_decode_bf16(qkv: torch.Tensor, q_stride: int, out: torch.Tensor, kcache: torch.Tensor,
                          vcache: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor,
                          num_seqs: int, max_seq_len: int, nq: int, nkv: int, d: int, window: int,
                          scale: float, err: torch.Tensor, workspace: Optional[torch.Tensor] = None,
                          inv_freq: Optional[torch.Tensor] = None, rotary_dim: int = 0,
                          write_kv: bool = False, keep_first: int = 0, chunk: int = 0, softcap: float = 0.0,
                          sinks: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                          gate_per_head: bool = False, bias: Optional[torch.Tensor] = None,
                          magnitude: float = 1.0, slopes: Optional[torch.Tensor] = None) -> None:
    """Split-KV tensor-core attention of sequences 0 .. num_seqs-1, one query token
    each: row s of ``qkv`` holds the token's q heads (and behind them its k and v
    heads if ``write_kv``), row s of ``out`` gets the result.  ``rotary_dim`` > 0
    rotates q (and the new k) in the kernel; ``write_kv`` stores the token's k and
    v into the cache in the kernel.  ``max_seq_len`` bounds every length.  The
    workspace (float32, ``attention_decode_workspace`` elements) holds the splits'
    partial results; it is allocated here if not given.  ``keep_first``, ``chunk``, ``softcap``, ``sinks`` and
    ``gate`` as in ``attention_simt_kv`` (gate: a row per sequence).  With any of them, and the rotation and
    cache write in the kernel, ``bias`` (float32 over a row's q, k and v heads) is added first and cosine and sine
    are multiplied by ``magnitude``, as ``head_norm_kv_write`` does for prompt portions."""
    lib = build.load_library("attention_mma")
    _contig(out, "out"); _contig(kcache, "kcache"); _contig(vcache, "vcache"); _contig(block_table, "block_table")
    assert qkv.dtype is torch.bfloat16 and kcache.dtype is torch.bfloat16 and out.dtype is torch.bfloat16
    need = attention_decode_workspace(num_seqs, nq, d, max_seq_len)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.float32, device=qkv.device)
    assert workspace.dtype is torch.float32 and workspace.numel() >= need
    if rotary_dim:
        assert inv_freq is not None and inv_freq.dtype is torch.float64 and inv_freq.numel() == rotary_dim // 2
    counters = _counters_for(qkv.device, num_seqs * nkv)
    if keep_first or chunk or softcap or sinks is not None or gate is not None or bias is not None or \
            magnitude != 1.0 or slopes is not None:
        gate_mode = _attention_opts_asserts(sinks, gate, gate_per_head, nq, d, slopes)
        if bias is not None:
            assert write_kv and bias.dtype is torch.float32 and bias.is_contiguous() and bias.numel() == (nq + 2 * nkv) * d
        _check(lib.rllm_attention_decode_bf16_opts(
            _ptr(qkv), c_int(q_stride), _ptr(out), _ptr(kcache), _ptr(vcache), _ptr(block_table),
            c_int(block_table.shape[1]), _ptr(seq_lens), c_int(num_seqs), c_int(max_seq_len), c_int(nq), c_int(nkv),
            c_int(d), c_int(kcache.shape[2]), c_int(kcache.shape[0]), c_int(window), c_float(scale), c_int(keep_first),
            c_int(chunk), c_float(softcap), _ptr(sinks), _ptr(gate), c_int(gate.stride(0) if gate is not None else 0),
            c_int(gate_mode), _ptr(inv_freq if rotary_dim else None), c_int(rotary_dim), c_int(1 if write_kv else 0),
            _ptr(bias), c_float(magnitude), _ptr(slopes), _ptr(workspace), _ptr(counters), _ptr(err), _stream()),
            "attention_decode_bf16_opts")
        return
    _check(lib.rllm_attention_decode_bf16(_ptr(qkv), c_int(q_stride), _ptr(out), _ptr(kcache), _ptr(vcache),
                                          _ptr(block_table), c_int(block_table.shape[1]), _ptr(seq_lens),
                                          c_int(num_seqs), c_int(max_seq_len), c_int(nq), c_int(nkv), c_int(d),
                                          c_int(kcache.shape[2]), c_int(kcache.shape[0]), c_int(window),
                                          c_float(scale), _ptr(inv_freq), c_int(rotary_dim),
                                          c_int(1 if write_kv else 0), _ptr(workspace), _ptr(counters),
                                          _ptr(err), _stream()), "attention_decode_bf16")


def attention_decode_workspace(num_seqs: int, nq: int, d: int, max_seq_len: int) -> int:
    lib = build.load_library("attention_mma")
    lib.rllm_attention_decode_workspace.restype = c_longlong
    return int(lib.rllm_attention_decode_workspace(c_int(num_seqs), c_int(nq), c_int(d), c_int(max_seq_len)))


def mma_attention_takes(nq: int, nkv: int, d: int) -> bool:
    return d in (16, 32, 64, 128) and nq % nkv == 0 and nq // nkv <= 16


def use_mma_attention(dtype: torch.dtype, nq: int, nkv: int, d: int) -> bool:
    """bfloat16 with a head size the tensor-core attention kernels take; other
    cases (float32, other head sizes) go to the CUDA-core kernel."""
    import os
    return dtype is torch.bfloat16 and mma_attention_takes(nq, nkv, d) and os.environ.get("RLLM_ATTENTION") != "simt"


def use_tcgen05_attention(dtype: torch.dtype, nq: int, nkv: int, d: int, page_size: int) -> bool:
    """Prompt portions go to the tcgen05 attention kernel when it takes the sizes;
    RLLM_ATTENTION=mma (or simt) keeps them on the older kernels."""
    import os
    return (dtype is torch.bfloat16 and attention_prefill_tcgen05_supported(nq, nkv, d, page_size)
            and os.environ.get("RLLM_ATTENTION") not in ("simt", "mma"))


def decode_advance(token_ids: torch.Tensor, positions: torch.Tensor, seq_lens: torch.Tensor,
                   sampled: torch.Tensor, history_row: Optional[torch.Tensor], count: Optional[int] = None) -> None:
    """For the first ``count`` rows (all by default): token_ids = sampled; positions += 1; seq_lens += 1;
    history_row = sampled.  ``history_row`` may be pinned host memory: the kernel then writes the tokens
    where the host reads them, and no copy stands in the stream."""
    lib = build.load_library("elementwise")
    n = token_ids.numel() if count is None else int(count)
    assert n <= token_ids.numel() and n <= sampled.numel() and (history_row is None or n <= history_row.numel())
    if history_row is not None and not history_row.is_cuda:
        # page-locked host memory has the same address on the device
        if not history_row.is_pinned() or history_row.dtype is not torch.int32:
            raise KernelError("decode_advance: a host row must be pinned int32 memory")
        row = c_void_p(history_row.data_ptr())
    else:
        row = _ptr(history_row)
    _check(lib.rllm_decode_advance(_ptr(token_ids), _ptr(positions), _ptr(seq_lens), _ptr(sampled),
                                   row, c_int(n), _stream()), "decode_advance")


def logprobs(logits: torch.Tensor, tokens: torch.Tensor, top_n: int):
    """Natural-log probabilities from raw logits float32 [R, V]: (lp [R] of ``tokens`` int32 [R], ids int32
    [R, top_n] and values float32 [R, top_n] of every row's ``top_n`` likeliest tokens, descending, the lower
    index first among equals; id -1 where nothing is left)."""
    lib = build.load_library("sampling")
    R, V = logits.shape
    assert logits.dtype is torch.float32 and logits.stride(1) == 1 and tokens.dtype is torch.int32 and tokens.numel() == R
    lp = torch.empty(R, dtype=torch.float32, device=logits.device)
    ids = torch.empty((R, top_n), dtype=torch.int32, device=logits.device)
    vals = torch.empty((R, top_n), dtype=torch.float32, device=logits.device)
    _check(lib.rllm_logprobs(_ptr(logits), c_int(R), c_int(V), c_int(logits.stride(0)), _ptr(tokens), c_int(top_n),
                             _ptr(lp), _ptr(ids) if top_n else c_void_p(0), _ptr(vals) if top_n else c_void_p(0),
                             _stream()), "logprobs")
    return lp, ids, vals


# ---------------------------------------------------------------------------
# gated, normalised sublayer results and the depth-weighted stream (layer_glue.cu)
# ---------------------------------------------------------------------------
def gated_postnorm_add(x_in: torch.Tensor, x_out: torch.Tensor, y: torch.Tensor, gate: Optional[torch.Tensor],
                       gate_bias: Optional[torch.Tensor], norm_weight: torch.Tensor, eps: float,
                       slot_weights: Optional[torch.Tensor] = None,
                       next_weight: Optional[torch.Tensor] = None, next_eps: float = 0.0,
                       depth=None) -> Optional[torch.Tensor]:
    """x_out = x_in + rmsnorm(v) * norm_weight with v = y * sigmoid(gate + gate_bias); x float32 [T, H]
    (x_out may be x_in; ``gate`` None: v = y, no gate).  ``slot_weights`` float32 [T, K]: y is [T * K, H] and a token's K rows are added
    with these factors first.  ``gate`` [T, H] may be a column slice (row stride >= H).  With
    ``next_weight`` the RMS norm of the new x under that weight is returned in the activation dtype.
    ``depth`` = (history float32 [L, T, H] whose level ``levels - 1`` is ``x_out``, levels, coeff [levels],
    stream_out float32 [T, H]): the depth average sum_j coeff[j] history[j] is written to ``stream_out`` in the
    same kernel, and the returned norm is the norm of that sum."""
    lib = build.load_library("layer_glue")
    T, H = x_in.shape
    hist = coeff = stream_out = None
    level_stride = levels = 0
    if depth is not None:
        hist, levels, coeff, stream_out = depth
        assert hist.dtype is torch.float32 and hist.is_contiguous() and hist.shape[1:] == (T, H) and 1 <= levels <= hist.shape[0]
        assert x_out.data_ptr() == hist[levels - 1].data_ptr() and coeff.numel() == levels and coeff.is_contiguous()
        assert coeff.dtype is norm_weight.dtype and stream_out.dtype is torch.float32 and stream_out.shape == (T, H)
        _contig(stream_out, "stream_out")
        level_stride = hist.stride(0)
    assert x_in.dtype is torch.float32 and x_out.dtype is torch.float32 and x_out.shape == x_in.shape
    _contig(x_in, "x_in"); _contig(x_out, "x_out"); _contig(y, "y")
    slots = 1
    if slot_weights is not None:
        assert slot_weights.dtype is torch.float32 and slot_weights.shape[0] == T
        _contig(slot_weights, "slot_weights")
        slots = slot_weights.shape[1]
    assert y.shape == (T * slots, H) and norm_weight.numel() == H
    if gate is not None:
        assert gate.shape == (T, H) and gate.dtype is y.dtype and gate.stride(1) == 1
        assert gate_bias.dtype is norm_weight.dtype and gate_bias.numel() == H
    g_stride = 0 if gate is None else (gate.stride(0) if T > 1 else max(H, gate.stride(0)))
    nxt = None
    if next_weight is not None:
        assert next_weight.dtype is norm_weight.dtype and next_weight.numel() == H
        nxt = torch.empty((T, H), dtype=y.dtype, device=y.device)
    _check(lib.rllm_gated_postnorm_add(_ptr(x_in), _ptr(x_out), _ptr(y), c_int(slots), _ptr(slot_weights),
                                       _ptr(gate), c_int(g_stride), _ptr(gate_bias if gate is not None else None), _ptr(norm_weight), c_float(eps), _ptr(next_weight),
                                       _ptr(nxt), c_float(next_eps), _ptr(hist), c_longlong(level_stride),
                                       c_int(levels), _ptr(coeff), _ptr(stream_out), c_int(T), c_int(H),
                                       c_int(dtype_code(y.dtype)), c_int(dtype_code(norm_weight.dtype)),
                                       _stream()), "gated_postnorm_add")
    return nxt


def depth_average(history: torch.Tensor, levels: int, coeff: torch.Tensor, stream_out: Optional[torch.Tensor],
                  norm_weight: Optional[torch.Tensor], eps: float, act_dtype: torch.dtype,
                  rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """s = sum_j coeff[j] * history[j] over the first ``levels`` levels; history float32 [L, T, H].
    Writes s to ``stream_out`` (float32 [T, H]) if given and returns rmsnorm(s) * norm_weight in
    ``act_dtype`` if a weight is given.  ``rows`` (int32 [R]): only these rows (no ``stream_out`` then)."""
    lib = build.load_library("layer_glue")
    L, T, H = history.shape
    assert history.dtype is torch.float32 and 1 <= levels <= L and coeff.numel() == levels
    _contig(history, "history"); _contig(coeff, "coeff")
    R = T if rows is None else rows.numel()
    if rows is not None:
        assert rows.dtype is torch.int32 and stream_out is None
    if stream_out is not None:
        assert stream_out.dtype is torch.float32 and stream_out.shape == (T, H)
        _contig(stream_out, "stream_out")
    out = None
    if norm_weight is not None:
        assert norm_weight.dtype is coeff.dtype and norm_weight.numel() == H
        out = torch.empty((R, H), dtype=act_dtype, device=history.device)
    _check(lib.rllm_depth_average(_ptr(history), c_longlong(history.stride(0)), c_int(levels), _ptr(coeff),
                                  _ptr(rows), _ptr(stream_out), _ptr(norm_weight), _ptr(out), c_float(eps),
                                  c_int(R), c_int(H), c_int(dtype_code(act_dtype)),
                                  c_int(dtype_code(coeff.dtype)), _stream()), "depth_average")
    return out


# ---------------------------------------------------------------------------
# minGRU (mingru.cu)
# ---------------------------------------------------------------------------
MINGRU_CHUNKED_FROM = 129      # a step whose longest portion has at least this many tokens scans in chunks


def mingru_scan(zxg: torch.Tensor, bias_z: torch.Tensor, bias_x: torch.Tensor, state: torch.Tensor,
                q_start: torch.Tensor, slots: torch.Tensor, num_seqs: int, out: torch.Tensor,
                err: torch.Tensor, max_q_len: int = 1) -> None:
    """zxg [T, >= 3 W]: a token's z, x and g projections side by side; state float32 [slots, W], updated in
    place for the sequences' slots; out [T, W] = S_t * silu(g).  ``max_q_len``: the most tokens a sequence
    brings; long portions are scanned in chunks of 64 that run side by side."""
    lib = build.load_library("mingru")
    T, W = out.shape
    if max_q_len >= MINGRU_CHUNKED_FROM and num_seqs * -(-max_q_len // 64) <= 65535:
        assert zxg.shape[0] == T and zxg.stride(1) == 1 and zxg.shape[1] >= 3 * W and out.dtype is zxg.dtype
        assert state.dtype is torch.float32 and state.shape[1] == W and bias_z.dtype is bias_x.dtype
        _contig(out, "out"); _contig(state, "state")
        chunks = -(-max_q_len // 64)
        work = torch.empty(num_seqs * chunks * 2 * W + num_seqs * W, dtype=torch.float32, device=out.device)
        _check(lib.rllm_mingru_scan_chunked(_ptr(zxg), c_int(zxg.stride(0)), _ptr(bias_z), _ptr(bias_x), _ptr(state),
                                            _ptr(q_start), _ptr(slots), c_int(state.shape[0]), _ptr(out),
                                            c_int(num_seqs), c_int(W), c_int(max_q_len), _ptr(work),
                                            c_int(dtype_code(out.dtype)), c_int(dtype_code(bias_z.dtype)),
                                            _ptr(err), _stream()), "mingru_scan_chunked")
        return
    assert zxg.shape[0] == T and zxg.stride(1) == 1 and zxg.shape[1] >= 3 * W and out.dtype is zxg.dtype
    assert state.dtype is torch.float32 and state.shape[1] == W
    assert bias_z.dtype is bias_x.dtype and bias_z.numel() == W and bias_x.numel() == W
    _contig(out, "out"); _contig(state, "state")
    _check(lib.rllm_mingru_scan(_ptr(zxg), c_int(zxg.stride(0)), _ptr(bias_z), _ptr(bias_x), _ptr(state),
                                _ptr(q_start), _ptr(slots), c_int(state.shape[0]), _ptr(out), c_int(num_seqs),
                                c_int(W), c_int(dtype_code(out.dtype)), c_int(dtype_code(bias_z.dtype)),
                                _ptr(err), _stream()), "mingru_scan")


# ---------------------------------------------------------------------------
# attention through a latent (latent_attention.cu)
# ---------------------------------------------------------------------------
def latent_prep(a: torch.Tensor, q_rank: int, kv_rank: int, rot: int, rot_dims: int, wq: torch.Tensor,
                wkv: Optional[torch.Tensor], eps: float, cq: torch.Tensor, cache: Optional[torch.Tensor],
                block_table: Optional[torch.Tensor], positions: torch.Tensor, token_seq: torch.Tensor,
                inv_freq: Optional[torch.Tensor], err: torch.Tensor, magnitude: float = 1.0) -> None:
    """a [T, q_rank (+ kv_rank + rot)]: the down projections of a token side by side.  cq [T, q_rank] =
    rmsnorm(a[:, :q_rank]) * wq.  With a cache ([pages, 1, page_size, kv_rank + rot]) the token's row is
    written: rmsnorm of the next kv_rank values times wkv, then the last rot values, the first rot_dims
    of them rotated by position (pairs 2i, 2i+1), cosine and sine times ``magnitude``."""
    lib = build.load_library("latent_attention")
    T = a.shape[0]
    write = cache is not None
    assert a.stride(1) == 1 and cq.shape == (T, q_rank) and cq.dtype is a.dtype
    _contig(cq, "cq")
    if write:
        assert a.shape[1] >= q_rank + kv_rank + rot and cache.dtype is a.dtype and cache.shape[3] == kv_rank + rot
        assert cache.shape[1] == 1 and wkv is not None and wkv.dtype is wq.dtype
        _contig(cache, "cache"); _contig(block_table, "block_table")
        if rot_dims:
            assert inv_freq is not None and inv_freq.dtype is torch.float64 and inv_freq.numel() == rot_dims // 2
        pages, page_size, max_blocks = cache.shape[0], cache.shape[2], block_table.shape[1]
    else:
        pages = page_size = max_blocks = 0
    _check(lib.rllm_latent_prep(_ptr(a), c_int(a.stride(0)), c_int(q_rank), c_int(kv_rank), c_int(rot),
                                c_int(rot_dims), _ptr(wq), _ptr(wkv), c_float(eps), _ptr(cq), _ptr(cache),
                                _ptr(block_table), c_int(max_blocks), _ptr(positions), _ptr(token_seq),
                                _ptr(inv_freq), c_float(magnitude), c_int(page_size), c_int(pages),
                                c_int(1 if write else 0),
                                c_int(T), c_int(dtype_code(a.dtype)), c_int(dtype_code(wq.dtype)), _ptr(err),
                                _stream()), "latent_prep")


def latent_q_rot(q: torch.Tensor, qt: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                 heads: int, dim: int, rot: int, rot_dims: int, kv_rank: int, magnitude: float = 1.0) -> None:
    """qt[t, h, kv_rank:] = q[t, h, dim:] with its first rot_dims values rotated by position (cosine and sine
    times ``magnitude``)."""
    lib = build.load_library("latent_attention")
    T = q.shape[0]
    assert q.shape == (T, heads * (dim + rot)) and qt.shape == (T, heads * (kv_rank + rot)) and qt.dtype is q.dtype
    _contig(q, "q"); _contig(qt, "qt")
    _check(lib.rllm_latent_q_rot(_ptr(q), _ptr(qt), _ptr(positions), _ptr(inv_freq), c_float(magnitude), c_int(T),
                                 c_int(heads),
                                 c_int(dim), c_int(rot), c_int(rot_dims), c_int(kv_rank),
                                 c_int(dtype_code(q.dtype)), _stream()), "latent_q_rot")


def head_gemm(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, b_kn: bool) -> None:
    """c[m, h, :] = a[m, h, :] . b[h] for every head h.  a [M, heads, K], c [M, heads, N]: views with unit
    stride in the last dim; b [heads, K, N] (``b_kn``) or [heads, N, K], contiguous."""
    lib = build.load_library("latent_attention")
    M, heads, K = a.shape
    N = c.shape[2]
    assert c.shape[:2] == (M, heads) and a.stride(2) == 1 and c.stride(2) == 1 and a.dtype is b.dtype is c.dtype
    assert b.shape == ((heads, K, N) if b_kn else (heads, N, K))
    _contig(b, "b")
    _check(lib.rllm_head_gemm(_ptr(a), c_longlong(a.stride(0)), c_longlong(a.stride(1)), _ptr(b),
                              c_longlong(b.stride(1)), c_longlong(b.stride(0)), c_int(1 if b_kn else 0), _ptr(c),
                              c_longlong(c.stride(0)), c_longlong(c.stride(1)), c_int(M), c_int(N), c_int(K),
                              c_int(heads), c_int(dtype_code(a.dtype)), _stream()), "head_gemm")


def latent_attention_simt(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                          positions: torch.Tensor, token_seq: torch.Tensor, heads: int, dk: int, dv: int,
                          window: int, scale: float, sink: Optional[torch.Tensor], err: torch.Tensor) -> None:
    """q [T, heads * dk], cache [pages, 1, page_size, dk], out [T, heads * dv]: softmax(q . row * scale) over
    the visible rows (``window`` 0: all up to the query's position), times the rows' first dv values.
    ``sink`` float32 [heads]: exp(sink[h]) joins the denominator."""
    lib = build.load_library("latent_attention")
    T = q.shape[0]
    assert q.shape == (T, heads * dk) and out.shape == (T, heads * dv) and cache.shape[3] == dk
    assert cache.dtype is q.dtype and out.dtype is q.dtype
    _contig(q, "q"); _contig(out, "out"); _contig(cache, "cache"); _contig(block_table, "block_table")
    if sink is not None:
        assert sink.dtype is torch.float32 and sink.numel() == heads
    _check(lib.rllm_latent_attention_simt(_ptr(q), _ptr(out), _ptr(cache), c_int(dtype_code(q.dtype)),
                                          _ptr(block_table), c_int(block_table.shape[1]), _ptr(positions),
                                          _ptr(token_seq), c_int(T), c_int(heads), c_int(dk), c_int(dv),
                                          c_int(cache.shape[2]), c_int(cache.shape[0]), c_int(window),
                                          c_float(scale), _ptr(sink), _ptr(err), _stream()),
           "latent_attention_simt")


LATENT_SPLIT_MAX_TILES = 64      # at most this many row tiles in a launch (they fill less than half the GPU) ...
LATENT_SPLIT_MIN_KEYS = 1024     # ... and at least this many keys to walk: the keys are cut into splits too
LATENT_SPLIT_KEYS = 128          # keys a split (a multiple of 64, at absolute positions)


def latent_attention_mma_takes(dtype: torch.dtype, dk: int, dv: int) -> bool:
    """Whether the tensor-core kernel computes this attention (RLLM_LATENT_ATTENTION=simt keeps it on the CUDA cores)."""
    import os
    return (dtype is torch.bfloat16 and dk % 8 == 0 and dv <= min(dk, 512)
            and os.environ.get("RLLM_LATENT_ATTENTION") != "simt")


def latent_attention_mma(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                         q_start: torch.Tensor, seq_lens: torch.Tensor, num_seqs: int, max_q_len: int, heads: int,
                         dk: int, dv: int, window: int, scale: float, sink: Optional[torch.Tensor],
                         err: torch.Tensor, max_seq_len: int = 0) -> None:
    """The same attention as ``latent_attention_simt`` on the tensor cores, for bfloat16.  Sequence s owns
    tokens q_start[s] .. q_start[s+1], the last of them at position seq_lens[s] - 1; ``max_q_len``: the most
    tokens a sequence brings (sizes the grid).  ``max_seq_len`` (an upper bound of seq_lens, 0: unknown): with
    few rows and long sequences the keys are also cut into splits of 128 that run side by side."""
    lib = build.load_library("latent_attention_mma")
    split_tiles, nsplit, work = 0, 1, None
    row_tiles = num_seqs * -(-(max_q_len * heads) // 64)
    keys = min(max_seq_len, window + max_q_len) if window else max_seq_len
    if row_tiles <= LATENT_SPLIT_MAX_TILES and keys >= LATENT_SPLIT_MIN_KEYS and max_seq_len <= 8192 * LATENT_SPLIT_KEYS:
        split_tiles = LATENT_SPLIT_KEYS                     # in keys: a multiple of every key tile
        nsplit = -(-max_seq_len // LATENT_SPLIT_KEYS)
        lib.rllm_latent_attention_mma_work.restype = c_longlong
        n = int(lib.rllm_latent_attention_mma_work(c_int(num_seqs), c_int(max_q_len), c_int(heads), c_int(dv),
                                                   c_int(nsplit)))
        work = torch.empty(n, dtype=torch.float32, device=q.device)
    T = q.shape[0]
    assert q.shape == (T, heads * dk) and out.shape == (T, heads * dv) and cache.shape[3] == dk
    assert q.dtype is torch.bfloat16 and cache.dtype is torch.bfloat16 and out.dtype is torch.bfloat16
    _contig(q, "q"); _contig(out, "out"); _contig(cache, "cache"); _contig(block_table, "block_table")
    if sink is not None:
        assert sink.dtype is torch.float32 and sink.numel() == heads
    _check(lib.rllm_latent_attention_mma(_ptr(q), _ptr(out), _ptr(cache), _ptr(block_table),
                                         c_int(block_table.shape[1]), _ptr(q_start), _ptr(seq_lens), c_int(num_seqs),
                                         c_int(max_q_len), c_int(heads), c_int(dk), c_int(dv), c_int(cache.shape[2]),
                                         c_int(cache.shape[0]), c_int(window), c_float(scale), _ptr(sink),
                                         c_int(split_tiles), c_int(nsplit), _ptr(work), _ptr(err), _stream()),
           "latent_attention_mma")


# ---------------------------------------------------------------------------
# routed experts (moe.cu)
# ---------------------------------------------------------------------------
MOE_SMALL_PAIRS = 64      # up to this many (token, expert) pairs a step the expert products use row tiles of 16


def moe_route(h: torch.Tensor, w_router: torch.Tensor, top: int):
    """(ids int32 [T, top], scores float32 [T, top]): softmax over all experts of the float32 logits
    h . w_router^T, the ``top`` largest in falling order (lowest index first among equals)."""
    lib = build.load_library("moe")
    T, H = h.shape
    E = w_router.shape[0]
    assert w_router.shape == (E, H) and w_router.dtype is h.dtype
    _contig(h, "h"); _contig(w_router, "w_router")
    ids = torch.empty((T, top), dtype=torch.int32, device=h.device)
    scores = torch.empty((T, top), dtype=torch.float32, device=h.device)
    _check(lib.rllm_moe_route(_ptr(h), _ptr(w_router), _ptr(ids), _ptr(scores), c_int(T), c_int(H), c_int(E),
                              c_int(top), c_int(dtype_code(h.dtype)), _stream()), "moe_route")
    return ids, scores


def moe_choose(logits: torch.Tensor, top: int, groups: int = 0, keep: int = 0, renormalise: bool = False):
    """``moe_route`` from router logits that a matrix product left in float32 [T, E].  ``groups`` > 0: the
    experts form that many equal groups of neighbours, a group's score is its largest expert score, and only
    experts of the ``keep`` best groups can be chosen.  ``renormalise``: the chosen scores are divided by their
    sum + 1e-20."""
    lib = build.load_library("moe")
    T, E = logits.shape
    assert logits.dtype is torch.float32
    _contig(logits, "logits")
    ids = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    scores = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    _check(lib.rllm_moe_choose(_ptr(logits), _ptr(ids), _ptr(scores), c_int(T), c_int(E), c_int(top), c_int(groups),
                               c_int(keep), c_int(1 if renormalise else 0), _stream()), "moe_choose")
    return ids, scores


def moe_experts(h: torch.Tensor, ids: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, limit: float,
                alpha: float, up_shift: float = 1.0) -> torch.Tensor:
    """out [T * top, H]: row t * top + k is expert ids[t, k] applied to h[t]:
    W_down (g' sigmoid(alpha g') (u' + up_shift)), g' = min(W_gate h, limit), u' = clamp(W_up h, +-limit)
    (limit inf, alpha 1, up_shift 0: silu(W_gate h) * W_up h).
    w_gate_up [E, 2 F, H] (gate rows, then up rows), w_down [E, H, F]."""
    lib = build.load_library("moe")
    T, H = h.shape
    top = ids.shape[1]
    E, F2, _ = w_gate_up.shape
    F = F2 // 2
    assert w_gate_up.shape == (E, 2 * F, H) and w_down.shape == (E, H, F) and ids.shape == (T, top)
    assert w_gate_up.dtype is h.dtype and w_down.dtype is h.dtype and ids.dtype is torch.int32
    _contig(h, "h"); _contig(w_gate_up, "w_gate_up"); _contig(w_down, "w_down"); _contig(ids, "ids")
    P = T * top
    bm = 16 if P <= MOE_SMALL_PAIRS else 64
    max_tiles = min(P, -(-P // bm) + E)
    meta = torch.empty(1 + (E + 1) + P + 2 * max_tiles, dtype=torch.int32, device=h.device)
    m_tiles, offsets, sorted_pairs = meta[0:1], meta[1:E + 2], meta[E + 2:E + 2 + P]
    tile_expert = meta[E + 2 + P:E + 2 + P + max_tiles]
    tile_row0 = meta[E + 2 + P + max_tiles:]
    _check(lib.rllm_moe_sort(_ptr(ids), c_int(P), c_int(E), c_int(bm), _ptr(offsets), _ptr(sorted_pairs),
                             _ptr(tile_expert), _ptr(tile_row0), _ptr(m_tiles), _stream()), "moe_sort")
    y = torch.empty((P, F), dtype=h.dtype, device=h.device)
    out = torch.empty((P, H), dtype=h.dtype, device=h.device)
    _check(lib.rllm_moe_experts(_ptr(h), _ptr(w_gate_up), _ptr(w_down), _ptr(y), _ptr(out), _ptr(offsets),
                                _ptr(sorted_pairs), _ptr(tile_expert), _ptr(tile_row0), _ptr(m_tiles),
                                c_int(max_tiles), c_int(bm), c_int(H), c_int(F), c_int(top), c_float(limit),
                                c_float(alpha), c_float(up_shift), c_int(dtype_code(h.dtype)), _stream()),
           "moe_experts")
    return out


def weighted_slot_sum(y: torch.Tensor, coeff: torch.Tensor, out: torch.Tensor, extra: Optional[torch.Tensor] = None,
                      extra_gate: Optional[torch.Tensor] = None) -> None:
    """out[t] = sum_k coeff[t, k] * y[t * K + k] (+ sigmoid(extra_gate[t]) * extra[t]); y [T * K, H], coeff
    float32 [T, K], out and extra [T, H], extra_gate float32 [T] (absent: the extra row is added as it is)."""
    lib = build.load_library("moe")
    T, H = out.shape
    K = coeff.shape[1]
    assert y.shape == (T * K, H) and coeff.shape == (T, K) and coeff.dtype is torch.float32 and y.dtype is out.dtype
    _contig(y, "y"); _contig(coeff, "coeff"); _contig(out, "out")
    if extra is not None:
        assert extra.shape == out.shape and extra.dtype is out.dtype
        _contig(extra, "extra")
        if extra_gate is not None:
            assert extra_gate.dtype is torch.float32 and extra_gate.numel() == T and extra_gate.is_contiguous()
    _check(lib.rllm_weighted_slot_sum(_ptr(y), _ptr(coeff), _ptr(out), c_int(T), c_int(K), c_int(H), _ptr(extra),
                                      _ptr(extra_gate if extra is not None else None),
                                      c_int(dtype_code(out.dtype)), _stream()), "weighted_slot_sum")


def moe_choose_sigmoid(logits: torch.Tensor, top: int, bias: Optional[torch.Tensor], scale: float):
    """(ids int32 [T, top], weights float32 [T, top]) from float32 router logits [T, E]: s = sigmoid(z); the
    ``top`` experts with the largest s + bias (float32 [E] or None; lowest index among equals), in falling
    order; weights s * scale without the bias."""
    lib = build.load_library("moe")
    T, E = logits.shape
    assert logits.dtype is torch.float32
    _contig(logits, "logits")
    if bias is not None:
        assert bias.dtype is torch.float32 and bias.numel() == E and bias.is_contiguous()
    ids = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    _check(lib.rllm_moe_choose_sigmoid(_ptr(logits), _ptr(bias), c_float(scale), _ptr(ids), _ptr(weights), c_int(T),
                                       c_int(E), c_int(top), _stream()), "moe_choose_sigmoid")
    return ids, weights


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}
PLAIN_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "relu_squared": 2}


def act(x: torch.Tensor, out: torch.Tensor, activation: str) -> None:
    """out = act(x) element by element (float32 arithmetic); act "silu", "gelu_tanh" or "relu_squared"
    (max(z, 0)^2); ``out`` may be ``x``."""
    lib = build.load_library("elementwise")
    assert x.shape == out.shape and x.dtype is out.dtype
    _contig(x, "x"); _contig(out, "out")
    _check(lib.rllm_act(_ptr(x), _ptr(out), c_int(dtype_code(out.dtype)), c_longlong(x.numel()),
                        c_int(PLAIN_ACTIVATIONS[activation]), _stream()), "act")


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = x[t, i] * sigmoid(gate[t, i]); gate may be a column slice (row stride >= its width)."""
    lib = build.load_library("elementwise")
    T, W = x.shape
    assert out.shape == x.shape and gate.shape == x.shape and gate.dtype is x.dtype and out.dtype is x.dtype
    assert gate.stride(1) == 1
    _contig(x, "x"); _contig(out, "out")
    _check(lib.rllm_sigmoid_gate(_ptr(x), _ptr(gate), c_int(gate.stride(0) if T > 1 else max(W, gate.stride(0))),
                                 _ptr(out), c_int(dtype_code(x.dtype)), c_int(T), c_int(W), _stream()), "sigmoid_gate")


def act_mul(gate_up: torch.Tensor, out: torch.Tensor, activation: str) -> None:
    """out[t, i] = act(gate_up[t, i]) * gate_up[t, I + i]; act "silu" or "gelu_tanh"."""
    lib = build.load_library("elementwise")
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and gate_up.dtype is out.dtype
    _contig(gate_up, "gate_up"); _contig(out, "out")
    _check(lib.rllm_act_mul(_ptr(gate_up), _ptr(out), c_int(dtype_code(out.dtype)), c_int(T), c_int(I),
                            c_int(ACTIVATIONS[activation]), _stream()), "act_mul")


# ---------------------------------------------------------------------------
# several residual streams (hyper_streams.cu)
# ---------------------------------------------------------------------------
HS_MAX_STREAMS = 8


def _norm_args(norm):
    """(alpha, weight, shift) of a dynamic-tanh norm, or three Nones."""
    if norm is None:
        return None, None, None
    alpha, w, c = norm
    assert alpha.dtype is torch.float32 and alpha.numel() == 1 and w.dtype is c.dtype and w.shape == c.shape
    _contig(w, "norm weight"); _contig(c, "norm shift")
    return alpha, w, c


def streams_read(xs: torch.Tensor, coeff: Optional[torch.Tensor], norm, out_dtype: torch.dtype,
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = n(sum_s coeff[s] * xs[s, row(r)]); xs float32 [S, T, H]; coeff float32 [S] (None: ones);
    ``norm`` = (alpha float32 [1], weight [H], shift [H]) applies n(u) = tanh(alpha u) * weight + shift and
    rounds to ``out_dtype``; None: out is the float32 sum.  ``rows`` int32 [R] picks rows."""
    lib = build.load_library("hyper_streams")
    S, T, H = xs.shape
    assert xs.dtype is torch.float32 and S <= HS_MAX_STREAMS
    _contig(xs, "xs")
    alpha, w, c = _norm_args(norm)
    if coeff is not None:
        assert coeff.dtype is torch.float32 and coeff.numel() == S and coeff.is_contiguous()
    R = T if rows is None else rows.numel()
    if rows is not None:
        assert rows.dtype is torch.int32
    od = out_dtype if w is not None else torch.float32
    out = torch.empty((R, H), dtype=od, device=xs.device)
    _check(lib.rllm_hs_read(_ptr(xs), _ptr(coeff), _ptr(rows), _ptr(alpha), _ptr(w), _ptr(c),
                            c_int(dtype_code(w.dtype) if w is not None else DT_F32), _ptr(out), c_int(dtype_code(od)),
                            c_int(S), c_longlong(T), c_int(R), c_int(H), _stream()), "streams_read")
    return out


def streams_write(xs: torch.Tensor, y: torch.Tensor, scale: Optional[torch.Tensor], mix: torch.Tensor,
                  write: torch.Tensor, next_read: Optional[torch.Tensor] = None, norm=None,
                  sum_out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """xs (float32 [S, T, H], in place): x_t <- sum_s mix[s, t] x_s + write[t] * (scale * y), all streams from
    the old ones; y [T, H]; scale [H] or None; mix float32 [S, S] (from, to); write float32 [S].  With
    ``next_read`` (float32 [S]) the next read comes back too: n(sum_t next_read[t] x_t) with ``norm`` as in
    ``streams_read`` (in y's dtype), or the float32 sum without one.  ``sum_out`` float32 [T, H], if given,
    receives the plain sum of the new streams."""
    lib = build.load_library("hyper_streams")
    S, T, H = xs.shape
    assert xs.dtype is torch.float32 and S <= HS_MAX_STREAMS and y.shape == (T, H)
    assert mix.dtype is torch.float32 and mix.shape == (S, S) and write.dtype is torch.float32 and write.numel() == S
    _contig(xs, "xs"); _contig(y, "y"); _contig(mix, "mix"); _contig(write, "write")
    alpha, w, c = _norm_args(norm)
    wd = w.dtype if w is not None else (scale.dtype if scale is not None else torch.float32)
    if scale is not None:
        assert scale.numel() == H and scale.is_contiguous() and scale.dtype is wd
    out = None
    if next_read is not None:
        assert next_read.dtype is torch.float32 and next_read.numel() == S and next_read.is_contiguous()
        out = torch.empty((T, H), dtype=y.dtype if w is not None else torch.float32, device=xs.device)
    if sum_out is not None:
        assert sum_out.dtype is torch.float32 and sum_out.shape == (T, H) and sum_out.is_contiguous()
    _check(lib.rllm_hs_write(_ptr(xs), _ptr(y), c_int(dtype_code(y.dtype)), _ptr(scale), _ptr(mix), _ptr(write),
                             _ptr(next_read), _ptr(alpha), _ptr(w), _ptr(c), c_int(dtype_code(wd)), _ptr(out),
                             _ptr(sum_out), c_int(S), c_longlong(T), c_int(H), _stream()), "streams_write")
    return out


def dyt(x: torch.Tensor, alpha: torch.Tensor, weight: torch.Tensor, shift: torch.Tensor, out: torch.Tensor,
        delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None, writeback: bool = False) -> None:
    """out = tanh(alpha * (x [+ delta])) * weight + shift; x float32 [., H]; the arguments of ``rmsnorm``."""
    lib = build.load_library("hyper_streams")
    H, R = x.shape[-1], out.shape[0]
    assert x.dtype is torch.float32 and alpha.dtype is torch.float32 and weight.dtype is shift.dtype
    _contig(x, "x"); _contig(out, "out")
    if delta is not None:
        assert delta.dtype is out.dtype and delta.shape == x.shape
        _contig(delta, "delta")
    if rows is not None:
        assert rows.dtype is torch.int32 and rows.numel() == R
    _check(lib.rllm_dyt(_ptr(x), _ptr(delta), _ptr(rows), _ptr(alpha), _ptr(weight), _ptr(shift),
                        c_int(dtype_code(weight.dtype)), _ptr(out), c_int(dtype_code(out.dtype)), c_int(R), c_int(H),
                        c_int(1 if writeback else 0), _stream()), "dyt")


# ---------------------------------------------------------------------------
# steps around mixers (mixer_glue.cu)
# ---------------------------------------------------------------------------
def head_norm_kv_write(qkv: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor,
                       q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                       block_table: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, nq: int, nkv: int,
                       dk: int, dv: int, err: torch.Tensor, write_kv: bool = True,
                       q_out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                       inv_freq: Optional[torch.Tensor] = None, rotary_dim: int = 0, magnitude: float = 1.0,
                       unit_norm: bool = False, q_temp=None) -> None:
    """qkv [T, nq dk + nkv dk + nkv dv]: every query head (in place) and key head is divided by its root mean
    square and multiplied by the weight [dk] (None: left as it is); keys and values go to the token's place in
    kcache [pages, nkv, page, dkp] and vcache [pages, nkv, page, dvp].  Cache rows wider than the heads (dkp > dk,
    dvp > dv) are filled up with zeros; the queries then go to ``q_out`` [T, nq * dkp], filled up alike.
    ``bias`` float32 [nq dk + nkv dk + nkv dv] is added to every row first; ``inv_freq`` float64 [rotary_dim / 2]
    with ``rotary_dim`` > 0 rotates the first rotary_dim dims of every query and key head by the token's position
    (dimension i with i + rotary_dim / 2), cosine and sine times ``magnitude``.  ``unit_norm``: the heads are
    divided by their root mean square although there are no weights.  ``q_temp`` = (coef, every): a query at
    position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1).  Columns of qkv behind the
    value heads are left alone."""
    lib = build.load_library("mixer_glue")
    T = qkv.shape[0]
    assert qkv.shape[1] >= nq * dk + nkv * (dk + dv) and qkv.stride(1) == 1
    if bias is not None:
        assert bias.dtype is torch.float32 and bias.is_contiguous() and bias.numel() == nq * dk + nkv * (dk + dv)
    if rotary_dim:
        assert inv_freq is not None and inv_freq.dtype is torch.float64 and inv_freq.numel() == rotary_dim // 2
    dkp = q_out.shape[1] // nq if q_out is not None else dk
    dvp = dv
    if q_out is not None:
        assert q_out.shape == (T, nq * dkp) and q_out.dtype is qkv.dtype and q_out.is_contiguous()
    wd = q_weight.dtype if q_weight is not None else torch.float32
    if q_weight is not None:
        assert k_weight is not None and k_weight.dtype is wd and q_weight.numel() == dk and k_weight.numel() == dk
    if write_kv:
        dvp = vcache.shape[3]
        assert kcache.dtype is qkv.dtype and vcache.dtype is qkv.dtype and kcache.shape[3] == dkp and dvp >= dv
        _contig(kcache, "kcache"); _contig(vcache, "vcache"); _contig(block_table, "block_table")
        pages, page_size, max_blocks = kcache.shape[0], kcache.shape[2], block_table.shape[1]
    else:
        pages = page_size = max_blocks = 0
    _check(lib.rllm_head_norm_kv_write(_ptr(qkv), c_int(dtype_code(qkv.dtype)), c_int(qkv.stride(0)), _ptr(positions),
                                       _ptr(token_seq), _ptr(q_weight), _ptr(k_weight), c_int(dtype_code(wd)),
                                       c_float(eps), _ptr(block_table), c_int(max_blocks),
                                       _ptr(kcache if write_kv else None), _ptr(vcache if write_kv else None),
                                       c_int(T), c_int(nq), c_int(nkv if write_kv else 0), c_int(dk), c_int(dv),
                                       c_int(dkp), c_int(dvp), _ptr(q_out),
                                       c_int(page_size), c_int(pages), c_int(1 if write_kv else 0), _ptr(bias),
                                       _ptr(inv_freq if rotary_dim else None), c_int(rotary_dim), c_float(magnitude),
                                       c_int(1 if unit_norm else 0), c_float(q_temp[0] if q_temp else 0.0),
                                       c_int(int(q_temp[1]) if q_temp else 0),
                                       _ptr(err), _stream()), "head_norm_kv_write")


def attention_simt_kv(q: torch.Tensor, q_stride: int, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                      block_table: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor, nq: int, nkv: int,
                      window: int, scale: float, err: torch.Tensor, keep_first: int = 0, chunk: int = 0,
                      softcap: float = 0.0, sinks: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                      gate_per_head: bool = False, slopes: Optional[torch.Tensor] = None) -> None:
    """``attention_simt`` where keys [pages, nkv, page, dk] and values [pages, nkv, page, dv] have sizes of their
    own: q rows of nq * dk, out [T, nq * dv]; any dk, dv up to 256.  ``keep_first``: with a window, the first
    that many keys of a sequence stay visible; ``chunk``: only keys of the query's own chunk of positions are;
    ``softcap``: scores become softcap * tanh(score / softcap); ``sinks`` float32 [nq]: exp(sink) joins each
    head's softmax denominator; ``gate`` [T, nq] (``gate_per_head``) or [T, nq * dv], a view with the rows'
    stride: the result is multiplied by its sigmoid; ``slopes`` float32 [nq]: slopes[h] * (query position - key
    position) is taken off every score."""
    lib = build.load_library("attention_simt")
    T, dk, dv = out.shape[0], kcache.shape[3], vcache.shape[3]
    _contig(out, "out"); _contig(kcache, "kcache"); _contig(vcache, "vcache"); _contig(block_table, "block_table")
    assert kcache.dtype is q.dtype and vcache.dtype is q.dtype and out.dtype is q.dtype and out.shape[1] == nq * dv
    if sinks is not None:
        assert sinks.dtype is torch.float32 and sinks.numel() == nq and sinks.is_contiguous()
    if gate is not None:
        assert gate.dtype is q.dtype and gate.stride(1) == 1 and gate.shape == (T, nq if gate_per_head else nq * dv)
    _check(lib.rllm_attention_simt_kv(_ptr(q), c_int(q_stride), _ptr(out), _ptr(kcache), _ptr(vcache),
                                      c_int(dtype_code(q.dtype)), _ptr(block_table), c_int(block_table.shape[1]),
                                      _ptr(positions), _ptr(token_seq), c_int(T), c_int(nq), c_int(nkv), c_int(dk),
                                      c_int(dv), c_int(kcache.shape[2]), c_int(kcache.shape[0]), c_int(window),
                                      c_float(scale), c_int(keep_first), c_int(chunk), c_float(softcap), _ptr(sinks),
                                      _ptr(gate), c_int(gate.stride(0) if gate is not None else 0),
                                      c_int(0 if gate is None else (1 if gate_per_head else 2)), _ptr(slopes),
                                      _ptr(err), _stream()), "attention_simt_kv")


def rms_mean2(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, eps: float) -> torch.Tensor:
    """(rms(a) * wa + rms(b) * wb) / 2 row by row, rms(x) = x / sqrt(mean(x^2) + eps); a, b [T, H]."""
    lib = build.load_library("mixer_glue")
    T, H = a.shape
    assert b.shape == a.shape and b.dtype is a.dtype and wa.dtype is wb.dtype and wa.numel() == H and wb.numel() == H
    _contig(a, "a"); _contig(b, "b"); _contig(wa, "wa"); _contig(wb, "wb")
    out = torch.empty_like(a)
    _check(lib.rllm_rms_mean2(_ptr(a), _ptr(b), _ptr(wa), _ptr(wb), c_int(dtype_code(wa.dtype)), _ptr(out),
                              c_int(dtype_code(a.dtype)), c_int(T), c_int(H), c_float(eps), _stream()), "rms_mean2")
    return out


def gated_rmsnorm(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float,
                  out_dtype: torch.dtype) -> torch.Tensor:
    """rms(x) * weight * sigmoid(gate); x float32 [T, H]; gate [T, H] (a column slice of a wider tensor will do)."""
    lib = build.load_library("mixer_glue")
    T, H = x.shape
    assert x.dtype is torch.float32 and gate.shape == (T, H) and gate.stride(1) == 1 and gate.dtype is out_dtype
    _contig(x, "x"); _contig(weight, "weight")
    out = torch.empty((T, H), dtype=out_dtype, device=x.device)
    _check(lib.rllm_gated_rmsnorm(_ptr(x), _ptr(gate), c_int(gate.stride(0)), _ptr(weight),
                                  c_int(dtype_code(weight.dtype)), _ptr(out), c_int(dtype_code(out_dtype)), c_int(T),
                                  c_int(H), c_float(eps), _stream()), "gated_rmsnorm")
    return out


# ---------------------------------------------------------------------------
# recurrences with a state per request (lightning.cu, selective_scan.cu)
# ---------------------------------------------------------------------------
SCAN_CHUNKED_FROM = 129       # portions from this many tokens on are scanned as chunks side by side


def _chunks_for(lib_chunk: int, max_q_len: int, num_seqs: int) -> int:
    if max_q_len < SCAN_CHUNKED_FROM:
        return 0
    chunks = -(-max_q_len // lib_chunk)
    return chunks if num_seqs * chunks <= 65535 else 0


def lightning_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
                   q_start: torch.Tensor, slots: torch.Tensor, num_seqs: int, err: torch.Tensor,
                   max_q_len: int = 1) -> torch.Tensor:
    """Linear attention with a decay per head.  q, k [T, heads * d] and v [T, heads * dv] are column slices of
    one tensor (the projections before their silu); state float32 [slots, heads, d, dv], updated in place;
    returns o float32 [T, heads * dv]."""
    lib = build.load_library("lightning")
    heads, d, dv = state.shape[1:]
    T = q.shape[0]
    assert q.shape == (T, heads * d) and k.shape == q.shape and v.shape == (T, heads * dv)
    assert q.stride(0) == k.stride(0) == v.stride(0) and q.stride(1) == k.stride(1) == v.stride(1) == 1
    assert q.dtype is k.dtype is v.dtype and state.dtype is torch.float32 and decay.dtype is torch.float32
    assert decay.numel() == heads
    _contig(state, "state")
    out = torch.empty((T, heads * dv), dtype=torch.float32, device=q.device)
    chunks = _chunks_for(int(lib.rllm_lightning_chunk()), max_q_len, num_seqs)
    work = torch.empty(num_seqs * chunks * heads * d * dv, dtype=torch.float32, device=q.device) if chunks else None
    _check(lib.rllm_lightning_scan(_ptr(q), _ptr(k), _ptr(v), c_int(q.stride(0)), c_int(dtype_code(q.dtype)),
                                   _ptr(decay), _ptr(state), _ptr(work), _ptr(q_start), _ptr(slots),
                                   c_int(state.shape[0]), c_int(num_seqs), c_int(chunks), _ptr(out), c_int(heads),
                                   c_int(d), c_int(dv), _ptr(err), _stream()), "lightning_scan")
    return out


def causal_conv(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, tail: torch.Tensor,
                q_start: torch.Tensor, token_seq: torch.Tensor, slots: torch.Tensor, num_seqs: int,
                any_long: bool, err: torch.Tensor) -> torch.Tensor:
    """silu(bias + causal convolution per channel); x [T, E] (a column slice will do); weight [E, taps], the
    last column the current token's; tail float32 [slots, taps - 1, E]: a request's last inputs, read for the
    places before this step and moved on.  ``any_long``: some sequence brings more than one token."""
    lib = build.load_library("selective_scan")
    T, E = x.shape
    taps = weight.shape[1]
    assert weight.shape == (E, taps) and bias.numel() == E and weight.dtype is bias.dtype and x.stride(1) == 1
    assert tail.dtype is torch.float32 and tuple(tail.shape[1:]) == (max(taps - 1, 0), E)
    _contig(weight, "weight"); _contig(bias, "bias"); _contig(tail, "tail")
    out = torch.empty((T, E), dtype=x.dtype, device=x.device)
    _check(lib.rllm_causal_conv(_ptr(x), c_int(x.stride(0)), c_int(dtype_code(x.dtype)), _ptr(weight), _ptr(bias),
                                c_int(dtype_code(weight.dtype)), _ptr(tail), _ptr(q_start), _ptr(token_seq),
                                _ptr(slots), c_int(tail.shape[0]), c_int(num_seqs), c_int(1 if any_long else 0),
                                _ptr(out), c_int(T), c_int(E), c_int(taps), _ptr(err), _stream()), "causal_conv")
    return out


def selective_scan(xc: torch.Tensor, dt_raw: torch.Tensor, dt_bias: torch.Tensor, bc: torch.Tensor, b_off: int,
                   c_off: int, a_log: torch.Tensor, dskip: torch.Tensor, z: torch.Tensor, state: torch.Tensor,
                   q_start: torch.Tensor, slots: torch.Tensor, num_seqs: int, err: torch.Tensor,
                   max_q_len: int = 1) -> torch.Tensor:
    """The selective recurrence.  xc [T, E]: the convolution's output; dt_raw float32 [T, E]: the step
    projection before bias and softplus; bc [T, .]: B at columns b_off .. + N, C at c_off .. + N; a_log [E, N];
    dskip [E]; z [T, E] (a column slice will do); state float32 [slots, N, E], updated in place.  Returns
    (sum_n S C + dskip xc) * silu(z) as [T, E] in xc's dtype."""
    lib = build.load_library("selective_scan")
    T, E = xc.shape
    N = state.shape[1]
    assert state.dtype is torch.float32 and state.shape[2] == E and dt_raw.dtype is torch.float32
    assert dt_raw.shape == (T, E) and a_log.shape == (E, N) and dskip.numel() == E and dt_bias.numel() == E
    assert a_log.dtype is dskip.dtype is dt_bias.dtype and bc.dtype is xc.dtype and z.dtype is xc.dtype
    assert bc.stride(1) == 1 and z.stride(1) == 1 and z.shape == (T, E)
    assert 0 <= b_off and b_off + N <= bc.shape[1] and 0 <= c_off and c_off + N <= bc.shape[1]
    _contig(xc, "xc"); _contig(dt_raw, "dt_raw"); _contig(a_log, "a_log"); _contig(state, "state")
    out = torch.empty((T, E), dtype=xc.dtype, device=xc.device)
    chunks = _chunks_for(int(lib.rllm_scan_chunk()), max_q_len, num_seqs)
    work = torch.empty(num_seqs * chunks * (N + 1) * E, dtype=torch.float32, device=xc.device) if chunks else None
    work_dt = work[num_seqs * chunks * N * E:] if chunks else None
    _check(lib.rllm_selective_scan(_ptr(xc), _ptr(dt_raw), _ptr(dt_bias), _ptr(bc), c_int(bc.stride(0)), c_int(b_off),
                                   c_int(c_off), _ptr(a_log), _ptr(dskip), _ptr(z), c_int(z.stride(0)),
                                   c_int(dtype_code(xc.dtype)), c_int(dtype_code(a_log.dtype)), _ptr(state),
                                   _ptr(work), _ptr(work_dt), _ptr(q_start), _ptr(slots), c_int(state.shape[0]),
                                   c_int(num_seqs), c_int(chunks), _ptr(out), c_int(E), c_int(N), _ptr(err),
                                   _stream()), "selective_scan")
    return out


# ---------------------------------------------------------------------------
# layer norm over the float32 stream (layernorm.cu)
# ---------------------------------------------------------------------------
def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float, out: torch.Tensor,
              deltas=(), row_bias: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
              writeback: bool = False) -> None:
    """out = (v - mean) / sqrt(mean of squared deviations + eps) * weight + bias, row by row in float32, with
    v = x + the sum of ``deltas`` (up to two [T, H] in out's dtype) + ``row_bias`` (float32 [H], every row).
    ``writeback``: x becomes v.  ``rows`` int32 [R]: out[r] is made from row rows[r]."""
    lib = build.load_library("layernorm")
    H = x.shape[-1]
    R = rows.numel() if rows is not None else x.shape[0]
    assert x.dtype is torch.float32 and x.is_contiguous() and out.is_contiguous() and out.shape == (R, H)
    assert weight.dtype is torch.float32 and bias.dtype is torch.float32 and weight.numel() == H and bias.numel() == H
    deltas = tuple(deltas)
    assert len(deltas) <= 2
    for d in deltas:
        assert d.dtype is out.dtype and d.shape == x.shape and d.is_contiguous()
    if row_bias is not None:
        assert row_bias.dtype is torch.float32 and row_bias.numel() == H and row_bias.is_contiguous()
    d0 = deltas[0] if deltas else None
    d1 = deltas[1] if len(deltas) > 1 else None
    _check(lib.rllm_layernorm(_ptr(x), _ptr(d0), _ptr(d1), _ptr(row_bias), _ptr(rows), _ptr(weight), _ptr(bias),
                              _ptr(out), c_int(dtype_code(out.dtype)), c_int(R), c_int(H), c_float(eps),
                              c_int(1 if writeback else 0), _stream()), "layernorm")


def add_rows(x: torch.Tensor, deltas, row_bias: Optional[torch.Tensor] = None) -> None:
    """x (float32 [T, H]) += the sum of ``deltas`` (one or two [T, H]) + ``row_bias`` (float32 [H])."""
    lib = build.load_library("layernorm")
    deltas = tuple(deltas)
    assert 1 <= len(deltas) <= 2 and x.dtype is torch.float32 and x.is_contiguous()
    for d in deltas:
        assert d.shape == x.shape and d.is_contiguous() and d.dtype is deltas[0].dtype
    if row_bias is not None:
        assert row_bias.dtype is torch.float32 and row_bias.numel() == x.shape[1] and row_bias.is_contiguous()
    _check(lib.rllm_add_rows(_ptr(x), _ptr(deltas[0]), _ptr(deltas[1] if len(deltas) > 1 else None), _ptr(row_bias),
                             c_int(dtype_code(deltas[0].dtype)), c_int(x.shape[0]), c_int(x.shape[1]), _stream()),
           "add_rows")


def add_row_bias(y: torch.Tensor, bias: torch.Tensor) -> None:
    """y [T, N] (bfloat16 or float32) += ``bias`` (float32 [N]) on every row, in place."""
    lib = build.load_library("layernorm")
    assert y.dim() == 2 and y.is_contiguous() and bias.dtype is torch.float32 and bias.numel() == y.shape[1]
    _check(lib.rllm_add_row_bias(_ptr(y), _ptr(bias), c_int(dtype_code(y.dtype)), c_int(y.shape[0]),
                                 c_int(y.shape[1]), _stream()), "add_row_bias")


# ---------------------------------------------------------------------------
# the matrix memory (mlstm.cu)
# ---------------------------------------------------------------------------
def mlstm_state_size(d: int, dv: int) -> int:
    """float32 values a head keeps: S [d, dv], n [d] and the running maximum."""
    return d * dv + d + 1


MLSTM_CHUNK = 64               # tokens a chunk of the chunked scan (the kernel's ML_CHUNK)
MLSTM_CHUNKED_FROM = 129       # a step whose longest portion has at least this many tokens scans in chunks


def mlstm_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gates: torch.Tensor, bias_i: torch.Tensor,
               bias_f: torch.Tensor, cap: float, qscale: float, state: torch.Tensor, q_start: torch.Tensor,
               slots: torch.Tensor, num_seqs: int, heads: int, d: int, dv: int, err: torch.Tensor,
               q_lens=None) -> torch.Tensor:
    """The mLSTM recurrence over this step's tokens of every sequence, in order, from and into the sequences'
    state slots.  q, k [T, heads * d] and v [T, heads * dv]: column slices of one product's result (one row
    stride); gates float32 [T, 2 heads]: pre-activations of the input gates, then of the forget gates (the
    call turns them into the log gates in place);
    ``cap``: both are capped as cap * tanh(z / cap) (0: not); q is multiplied by ``qscale``.
    state float32 [slots, heads, d * dv + d + 1].  Returns o float32 [T, heads * dv].  ``q_lens`` (the
    sequences' token counts of this step, host integers): if the longest has ``MLSTM_CHUNKED_FROM`` tokens or
    more, the sequences are cut into chunks of ``MLSTM_CHUNK`` tokens that run side by side (three launches);
    the results differ from the token-by-token walk by rounding only."""
    lib = build.load_library("mlstm")
    T = q.shape[0]
    assert q.shape == (T, heads * d) and k.shape == (T, heads * d) and v.shape == (T, heads * dv)
    assert q.dtype is k.dtype and k.dtype is v.dtype and q.stride(0) == k.stride(0) == v.stride(0)
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1
    assert gates.dtype is torch.float32 and gates.shape == (T, 2 * heads) and gates.is_contiguous()
    assert bias_i.dtype is torch.float32 and bias_f.dtype is torch.float32 and bias_i.numel() == heads == bias_f.numel()
    assert state.dtype is torch.float32 and state.is_contiguous() and state.shape[1:] == (heads, mlstm_state_size(d, dv))
    out = torch.empty((T, heads * dv), dtype=torch.float32, device=q.device)
    chunks, local, start = 0, None, None
    if q_lens is not None and len(q_lens) == num_seqs and max(q_lens, default=0) >= MLSTM_CHUNKED_FROM:
        chunks = sum(-(-int(n) // MLSTM_CHUNK) for n in q_lens)
        per = mlstm_state_size(d, dv)
        if chunks > 65535:
            chunks = 0
        else:
            local = torch.empty((chunks, heads, per + 1), dtype=torch.float32, device=q.device)
            start = torch.empty((chunks, heads, per), dtype=torch.float32, device=q.device)
    _check(lib.rllm_mlstm_scan(_ptr(q), _ptr(k), _ptr(v), c_int(q.stride(0)), c_int(dtype_code(q.dtype)), _ptr(gates),
                               _ptr(bias_i), _ptr(bias_f), c_float(cap), c_float(qscale), _ptr(state), _ptr(q_start),
                               _ptr(slots), _ptr(out), c_int(T), c_int(num_seqs), c_int(heads), c_int(d), c_int(dv),
                               c_int(state.shape[0]), c_int(chunks), _ptr(local), _ptr(start), _ptr(err), _stream()),
           "mlstm_scan")
    return out


def head_gated_rmsnorm(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, heads: int,
                       out_dtype: torch.dtype) -> torch.Tensor:
    """out = x / sqrt(mean over a head's values of x^2 + eps) * weight * sigmoid(gate); x float32 [T, heads * dv],
    weight [heads * dv], gate [T, heads * dv] in ``out_dtype`` (may be a column slice)."""
    lib = build.load_library("mlstm")
    T, W = x.shape
    assert x.dtype is torch.float32 and x.is_contiguous() and W % heads == 0 and weight.numel() == W
    assert gate.shape == (T, W) and gate.dtype is out_dtype and gate.stride(1) == 1
    _contig(weight, "weight")
    out = torch.empty((T, W), dtype=out_dtype, device=x.device)
    _check(lib.rllm_head_gated_rmsnorm(_ptr(x), _ptr(gate), c_int(gate.stride(0) if T > 1 else max(W, gate.stride(0))),
                                       _ptr(weight), c_int(dtype_code(weight.dtype)), _ptr(out),
                                       c_int(dtype_code(out_dtype)), c_int(T), c_int(heads), c_int(W // heads),
                                       c_float(eps), _stream()), "head_gated_rmsnorm")
    return out
