"""The device operations of the engine: thin wrappers over the ``extern "C"`` launchers
of the CUDA library.  There is one implementation of each operation and no fallback:
without a CUDA device, nvcc-built library and sm_100-class GPU the first call raises.

Conventions: tensors are contiguous CUDA tensors; ``T`` is the compute dtype (bfloat16
or float32); the residual stream, norm scales, rotary tables and logits are float32;
integer metadata is int32.  Launches go to torch's current CUDA stream.
"""
from __future__ import annotations

import collections
import ctypes
import math
import os
from typing import Optional

import torch

from . import build as _build

_lib = None
ABI_VERSION = 4
#: launches of this library's kernels so far (library matrix products are not counted)
launches = 0
#: calls by kind, for tests that must know which kernel a product or an attention went to
#: ("gemm_skinny", "gemm_tc", "gemm_library", "attn_tc", "attn_keys", "attn_rows", ...)
calls: "collections.Counter[str]" = collections.Counter()


class KernelError(RuntimeError):
    pass


def library():
    """Load (building at the first call) the CUDA library; raise if that is impossible."""
    global _lib
    if _lib is not None:
        return _lib
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: this engine runs on hand-written sm_100a kernels only and has no "
                          "CPU path")
    major, _minor = torch.cuda.get_device_capability()
    if major != 10:
        raise KernelError(f"the kernels are built for sm_100a (B200); this device is sm_{major}{_minor}")
    path = _build.build()
    lib = ctypes.CDLL(path)
    lib.tis_last_error.restype = ctypes.c_char_p
    lib.tis_abi_version.restype = ctypes.c_int
    if lib.tis_abi_version() != ABI_VERSION:
        raise KernelError(f"{path}: launcher interface {lib.tis_abi_version()}, expected {ABI_VERSION}")
    _lib = lib
    return lib


def is_loaded() -> bool:
    return _lib is not None


def _check(status: int, lib) -> None:
    global launches
    if status != 0:
        raise KernelError(lib.tis_last_error().decode())
    launches += 1


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"unsupported dtype {t.dtype}")


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """torch's current CUDA stream as a raw handle (the direct getter is 40 times cheaper than going
    through a Stream object, and this runs once per launch)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _f(x: float):
    return ctypes.c_float(x)


# ---------------------------------------------------------------------------------------
# matrix products (library GEMMs, as upstream uses for every projection:
# main_models_new.py:20,29,226)
# ---------------------------------------------------------------------------------------

#: rows up to which bfloat16 products go to the weight-streaming kernels of this library instead of the library
#: product (and up to which a step's norms are folded into them).  Measured inside the decode step of the 0.9B model
#: on a B200, ms a step with the limit at 8 / 16: batch 10 1.467 / 1.387, batch 12 1.491 / 1.397, batch 16
#: 1.544 / 1.437; at 16 / 32: batch 24 2.045 / 1.986, batch 32 2.132 / 2.068; at 64 rows the library wins by far
#: (batch 64: 3.02 against 4.22 ms).  (Before the reductions of these kernels were pushed and the norms folded in,
#: the library won from 9 rows, and before that from 5.)  TIS_SKINNY_MAX_ROWS in the environment overrides it
#: (0 sends everything to the library; the kernels themselves take up to 64 rows).
SKINNY_MAX_ROWS = int(os.environ.get("TIS_SKINNY_MAX_ROWS", "32"))
#: the gate/up product with the gating in its epilogue saves a launch and the round trip of the
#: ungated product: the kernel keeps it up to more rows (measured alone at 8 rows: 8.4 us against 9.1 us
#: for the library product plus the gating kernel; inside the decode step at batch 8: 5123 -> 5207 tok/s)
SKINNY_SWIGLU_MAX_ROWS = int(os.environ.get("TIS_SKINNY_SWIGLU_MAX_ROWS", "16"))
#: above that and up to this many rows the gate/up product with the gating goes to the tcgen05 kernel with swapped
#: operands (csrc/gemm_swap.cu).  Measured alone at the 0.9B shapes: 9.9 us at 32 rows and 11.7 us at 64, against 10.4 and
#: 10.6 us for the library product, which still needs the gating kernel (~2.5 us) after it; the plain products of these
#: row counts stay with the library (qkv at 64 rows: 4.6 us against 7.8).  Inside the decode step of the 0.9B model:
#: batch 24 2.022 -> 2.012 ms, batch 32 2.135 -> 2.119, batch 64 3.052 -> 3.078, so it is used up to 32 rows.
#: TIS_SWAP_SWIGLU_MAX_ROWS overrides (0: never).
SWAP_SWIGLU_MAX_ROWS = int(os.environ.get("TIS_SWAP_SWIGLU_MAX_ROWS", "32"))
EPI_STORE, EPI_SWIGLU, EPI_RESIDUAL = 0, 1, 2
#: the norm between two weight-streaming products is folded into them (``ResidualSink`` / ``ScaledRows``);
#: TIS_FUSED_NORM=0 keeps the norm kernel
FUSED_NORM = os.environ.get("TIS_FUSED_NORM", "1") != "0"


#: the factor a norm multiplies a row with, as a function of the row's sum of squares s over a width d:
#: "l2_eps": sqrt(d) / (sqrt(s) + eps) (eps added to the L2 norm); "mean_eps": rsqrt(s / d + eps)
NORM_KINDS = {"l2_eps": 0, "mean_eps": 1}


class ResidualSink:
    """Where a product adds its result itself: the float32 residual stream ``values`` (n, d); it then also
    leaves the stream times ``weight`` (the weight of the norm that reads the stream next) and partial sums of
    squares, so that the norm's factor per row (``kind``, one of ``NORM_KINDS``) can be applied after the next
    product instead of before it.  ``norm`` is whoever made the sink (the reader checks it is the same norm)."""

    def __init__(self, values: torch.Tensor, weight: torch.Tensor, eps: float, norm=None, kind: str = "l2_eps"):
        if kind not in NORM_KINDS:
            raise KernelError(f"norm factor {kind!r}: the products know {sorted(NORM_KINDS)}")
        self.values, self.weight, self.eps, self.norm, self.kind = values, weight, float(eps), norm, kind


class ScaledRows:
    """Rows of a norm's output that still lack the factor of their row: ``rows`` (n, d) bfloat16 = stream *
    norm weight, ``parts`` (n, T) float32 = partial sums of squares of the stream.  Row r of the norm's
    output is ``rows[r]`` times the factor of ``kind`` (``NORM_KINDS``) at ``parts[r].sum()``; a weight-streaming
    product applies the factor to its own result (``gemm`` and ``gemm_swiglu`` take these rows), ``dense()`` makes
    the rows whole."""

    def __init__(self, rows: torch.Tensor, parts: torch.Tensor, eps: float, norm=None, kind: str = "l2_eps"):
        self.rows, self.parts, self.eps, self.norm, self.kind = rows, parts, float(eps), norm, kind

    @property
    def shape(self):
        return self.rows.shape

    @property
    def dtype(self):
        return self.rows.dtype

    def dense(self) -> torch.Tensor:
        lib = library()
        n, d = self.rows.shape
        out = torch.empty_like(self.rows)
        calls["scale_rows"] += 1
        _check(lib.tis_scale_rows(_p(self.rows), self.rows.stride(0), _p(self.parts), self.parts.shape[1], _f(self.eps),
                                  NORM_KINDS[self.kind], _p(out), out.stride(0), n, d, _stream()), lib)
        return out


def sink_usable(values: torch.Tensor, dtype: torch.dtype) -> bool:
    """Whether a step of these rows can fold its norms into the products around them: bfloat16 products of
    few enough rows that they all go to the weight-streaming kernels."""
    n, d = values.shape
    return (FUSED_NORM and dtype == torch.bfloat16 and 0 < n <= SKINNY_MAX_ROWS and d % 8 == 0
            and values.stride(1) == 1 and values.stride(0) % 2 == 0)


def _skinny_ok(a: torch.Tensor, w: torch.Tensor, max_rows: Optional[int] = None) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and 0 < a.shape[0] <= (SKINNY_MAX_ROWS if max_rows is None else max_rows)
            and w.stride(1) == 1 and a.stride(1) == 1 and a.shape[1] % 8 == 0 and w.shape[1] % 8 == 0
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0)


#: The ring kernel wins where a CTA's share of K is short: up to RING_MAX_TILES tiles of 64 rows.  With longer
#: shares (the products of larger models) the loop is what counts, and the TMA-fed tcgen05 kernel with swapped
#: operands streams better.  Measured alone on a B200 at 1..8 rows, us ring / library / swapped: 3B-sized model
#: (width 3072, ffn 8192) qkv (12 tiles a CTA) 11.2 / 7.3 / 9.8, o (6) 6.1 / 8.5 / 7.3, gate/up with gating (24)
#: 21.8 / 22.8 + gating / 19.0, down (16) 14.2 / 17.9 / 12.6; 8B-sized (4096, 14336) qkv (16) 14.4 / 10.0 / 12.3,
#: o (8) 8.9 / 13.5 / 9.6, gate/up (64) 57 / 40 + gating / 38, down (28) 24.4 / 22.9 / 20.9.  So: short shares to the
#: ring; long ones to the swapped kernel when the matrix is tall (K >= 2 N) or carries the gating, else to the library.
RING_MAX_TILES = int(os.environ.get("TIS_RING_MAX_TILES", "8"))


def _ring_tiles(n_cols: int, k: int) -> int:
    """Tiles of 64 rows of K that a CTA of the ring kernel walks."""
    return -(-(-(-k // _ksplit(n_cols, k))) // 64)


def _swap_ok(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, swiglu: bool = False) -> bool:
    return (a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and (not swiglu or w.shape[1] % 64 == 0)
            and (out is None or out.stride(1) == 1))


def _ksplit(n_cols: int, k: int) -> int:
    """CTAs that share a 64-column strip of the weights (a cluster adding up over K): as many as
    keep the grid near two CTAs per SM, each with at least 128 rows of K."""
    strips = (n_cols + 63) // 64
    ks = 8
    while ks > 1 and (strips * ks > 2 * 148 * 2 or k // ks < 128):
        ks //= 2
    return ks


#: The weight-streaming product comes in two kernels: weights copied by the threads into a ring of four
#: stages (csrc/gemm_skinny.cu), and weights ordered as TMA boxes, a CTA's whole share of K at once
#: (csrc/gemm_stream.cu).  Measured alone on a B200 at the 0.9B shapes (us at 1 / 8 / 16 rows; library beside):
#: qkv 4.1 / 4.4 / 4.6 ring, 5.2 / 5.8 / 6.3 boxes (4.8 / 4.8 / 4.5); gate/up with gating 7.6 / 8.3 / 9.1 ring,
#: 10.9 / 11.9 / 13.5 boxes; down (K 4096, 512 rows of K a CTA) 7.4 / 7.8 / 8.2 ring, 6.2 / 6.5 / 6.9 boxes
#: (7.4 / 7.4 / 7.4).  A box row is 128 bytes, one request of the TMA engine each: with many CTAs per SM the
#: engine is the bottleneck, while a long share of K gains from having all of it in flight from the start.  With
#: shares of more than one round of boxes (the 3B- and 8B-sized models: 1024 rows of K a CTA and more) the kernel
#: loses to both others (8B model at one row: 132 against 210 tok/s).  So the boxes take products whose share of
#: K per CTA is STREAM_MIN_KC..STREAM_MAX_KC rows (one full round), of at most STREAM_MAX_CTAS CTAs, up to
#: STREAM_MAX_ROWS rows of x.
STREAM_GEMM = os.environ.get("TIS_STREAM_GEMM", "1") != "0"
STREAM_MIN_KC = int(os.environ.get("TIS_STREAM_MIN_KC", "512"))
STREAM_MAX_KC = int(os.environ.get("TIS_STREAM_MAX_KC", "512"))
STREAM_MAX_CTAS = int(os.environ.get("TIS_STREAM_MAX_CTAS", "296"))
STREAM_MAX_ROWS = int(os.environ.get("TIS_STREAM_MAX_ROWS", "32"))


def _stream_pays(n: int, k: int, cols: int, ksplit: Optional[int] = None) -> bool:
    ks = ksplit or _ksplit(cols, k)
    kc = -(-k // ks)
    return (STREAM_GEMM and n <= STREAM_MAX_ROWS and STREAM_MIN_KC <= kc <= max(STREAM_MAX_KC, STREAM_MIN_KC)
            and -(-cols // 64) * ks <= STREAM_MAX_CTAS)


def _ksplit_swap(n_cols: int, k: int) -> int:
    """CTAs that share a strip of 128 columns in the tcgen05 product with swapped operands."""
    strips = (n_cols + 127) // 128
    ks = 8
    while ks > 1 and (strips * ks > 2 * 148 or k // ks < 128):
        ks //= 2
    return ks


def gemm_swap(a, w: torch.Tensor, out: Optional[torch.Tensor] = None, swiglu: bool = False,
              ksplit: Optional[int] = None, sink: Optional["ResidualSink"] = None):
    """``a (n <= 64, K) @ w (K, N)`` in bfloat16 on the tcgen05 tensor cores with the operands swapped (128
    columns of ``w`` are the rows of the tile, the rows of ``a`` its narrow side); with ``swiglu`` the columns of
    ``w`` are [32 gate | 32 up] blocks and the result is (n, N/2).  ``a`` may be ``ScaledRows``; with ``sink`` the
    result is added to the residual stream and comes back as ``ScaledRows``."""
    lib = library()
    scaled = a if isinstance(a, ScaledRows) else None
    if scaled is not None:
        a = scaled.rows
    n, k = a.shape
    cols = w.shape[1]
    if not _sink_fits(sink, n, cols, out) or (sink is not None and swiglu):
        raise KernelError("gemm_swap: the sink does not fit the product")
    head, tail, result = _fused_args(scaled, sink, n, cols, a.device)
    if sink is not None:
        out = result.rows
    elif out is None:
        out = torch.empty((n, cols // 2 if swiglu else cols), dtype=a.dtype, device=a.device)
    calls["gemm_swap"] += 1
    epi = EPI_RESIDUAL if sink is not None else (EPI_SWIGLU if swiglu else EPI_STORE)
    _check(lib.tis_gemm_swap_fused(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), out.stride(0), n, cols, k,
                                   ksplit or _ksplit_swap(cols, k), epi, *head, *tail, _p(tc_fault()), _stream()), lib)
    return result if sink is not None else out


def _stream_fits(n: int, k: int, ksplit: int) -> bool:
    """Whether a CTA's share of the rows (all of its share of K, in shared memory for the whole loop) and
    a round of weight boxes fit the TMA-fed kernel's shared memory."""
    kc = -(-(-(-k // ksplit)) // 64) * 64
    rows = 16 if n <= 16 else (32 if n <= 32 else 64)
    received = ksplit * -(-rows // ksplit) * 64 * 4          # partial sums pushed by the cluster
    return min(kc // 64, 8) * 8192 + rows * (kc + 8) * 2 + received + 1024 <= 224 * 1024


def _fused_args(scaled: Optional[ScaledRows], sink: Optional[ResidualSink], n: int, cols: int, device):
    """The arguments of the fused entry points after (ksplit, epi): the partial sums of the rows, and the
    sink with the tensors it fills."""
    result = None
    if scaled is not None:
        head = (_p(scaled.parts), scaled.parts.shape[1], _f(scaled.eps), scaled.rows.shape[1], NORM_KINDS[scaled.kind])
    else:
        head = (None, 0, _f(0.0), 0, 0)
    if sink is not None:
        parts = torch.empty((n, -(-cols // 64)), dtype=torch.float32, device=device)
        rows = torch.empty((n, cols), dtype=torch.bfloat16, device=device)
        result = ScaledRows(rows, parts, sink.eps, sink.norm, sink.kind)
        tail = (_p(sink.values), sink.values.stride(0), _p(sink.weight), _p(parts))
    else:
        tail = (None, 0, None, None)
    return head, tail, result


def _sink_fits(sink: Optional[ResidualSink], n: int, cols: int, out) -> bool:
    return sink is None or (out is None and tuple(sink.values.shape) == (n, cols) and sink.weight.shape[0] == cols
                            and sink.weight.dtype == torch.float32 and sink.values.dtype == torch.float32)


def gemm_stream(a, w: torch.Tensor, out: Optional[torch.Tensor] = None, swiglu: bool = False,
                ksplit: Optional[int] = None, sink: Optional[ResidualSink] = None):
    """``a (n <= 64, K) @ w (K, N)`` in bfloat16 by the TMA-fed weight-streaming kernel; with ``swiglu``
    the columns of ``w`` are [32 gate | 32 up] blocks and the result is (n, N/2).  ``a`` may be ``ScaledRows``;
    with ``sink`` the result is added to the residual stream and comes back as ``ScaledRows``."""
    lib = library()
    scaled = a if isinstance(a, ScaledRows) else None
    if scaled is not None:
        a = scaled.rows
    n, k = a.shape
    cols = w.shape[1]
    if not _sink_fits(sink, n, cols, out) or (sink is not None and swiglu):
        raise KernelError("gemm_stream: the sink does not fit the product")
    head, tail, result = _fused_args(scaled, sink, n, cols, a.device)
    if sink is not None:
        out = result.rows
    elif out is None:
        out = torch.empty((n, cols // 2 if swiglu else cols), dtype=a.dtype, device=a.device)
    calls["gemm_stream"] += 1
    epi = EPI_RESIDUAL if sink is not None else (EPI_SWIGLU if swiglu else EPI_STORE)
    _check(lib.tis_gemm_stream_fused(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), out.stride(0), n, cols, k,
                                     ksplit or _ksplit(cols, k), epi, *head, *tail, _p(tc_fault()), _stream()), lib)
    return result if sink is not None else out


def gemm_skinny(a, w: torch.Tensor, out: Optional[torch.Tensor] = None, swiglu: bool = False,
                ksplit: Optional[int] = None, sink: Optional[ResidualSink] = None):
    """``a (n <= 64, K) @ w (K, N)`` in bfloat16 by a weight-streaming kernel; with ``swiglu``
    the columns of ``w`` are [32 gate | 32 up] blocks and the result is (n, N/2).  ``a`` may be ``ScaledRows``;
    with ``sink`` the result is added to the residual stream and comes back as ``ScaledRows``."""
    rows = a.rows if isinstance(a, ScaledRows) else a
    if (_stream_pays(rows.shape[0], rows.shape[1], w.shape[1], ksplit) and rows.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and _stream_fits(rows.shape[0], rows.shape[1], ksplit or _ksplit(w.shape[1], rows.shape[1]))):
        return gemm_stream(a, w, out, swiglu, ksplit, sink)
    lib = library()
    scaled = a if isinstance(a, ScaledRows) else None
    a = rows
    n, k = a.shape
    cols = w.shape[1]
    if not _sink_fits(sink, n, cols, out) or (sink is not None and swiglu):
        raise KernelError("gemm_skinny: the sink does not fit the product")
    head, tail, result = _fused_args(scaled, sink, n, cols, a.device)
    if sink is not None:
        out = result.rows
    elif out is None:
        out = torch.empty((n, cols // 2 if swiglu else cols), dtype=a.dtype, device=a.device)
    calls["gemm_skinny"] += 1
    epi = EPI_RESIDUAL if sink is not None else (EPI_SWIGLU if swiglu else EPI_STORE)
    _check(lib.tis_gemm_skinny_fused(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), out.stride(0), n, cols, k,
                                     ksplit or _ksplit(cols, k), epi, *head, *tail, _p(tc_fault()), _stream()), lib)
    return result if sink is not None else out


#: The tcgen05 kernel of this library (csrc/gemm_tc.cu) against the library product, measured on a
#: B200 at the 0.9B model's shapes (replayed from CUDA graphs, weights rotated through more than L2):
#: gate/up with the SwiGLU gating in its epilogue it wins from about 3000 rows (4096 rows: 78 against
#: 94 us for the library product plus the gating kernel; 2048 rows: 52 against 49 us); plain products
#: it loses (2048 x 1536 x 4096: 28 against 19.5 us — one CTA per tile moves more bytes from L2 per
#: multiply-add than the library's two-CTA tiles).  So by default it takes gate/up products of at
#: least TC_MIN_ROWS rows and no plain ones; TIS_TC_MIN_ROWS / TIS_TC_PLAIN_MIN_ROWS in the
#: environment override the two limits (0 = never).
TC_MIN_ROWS = int(os.environ.get("TIS_TC_MIN_ROWS", "3072"))
TC_PLAIN_MIN_ROWS = int(os.environ.get("TIS_TC_PLAIN_MIN_ROWS", "0"))
_tc_fault = None


def tc_fault() -> torch.Tensor:
    """The fault word of the tcgen05 products (non-zero after a wait inside one ran out)."""
    global _tc_fault
    if _tc_fault is None:
        _tc_fault = torch.zeros(4, dtype=torch.int32, device="cuda")
    return _tc_fault


def _tc_ok(a: torch.Tensor, w: torch.Tensor, min_rows: int) -> bool:
    return (min_rows > 0 and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and a.shape[0] >= min_rows and w.stride(1) == 1 and a.stride(1) == 1
            and a.shape[1] % 8 == 0 and w.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, swiglu: bool = False) -> torch.Tensor:
    """``a (n, K) @ w (K, N)`` in bfloat16 on the tcgen05 tensor cores (TMA-fed, accumulator in
    tensor memory); with ``swiglu`` the columns of ``w`` are [32 gate | 32 up] blocks and the
    result is (n, N/2)."""
    lib = library()
    n, k = a.shape
    cols = w.shape[1]
    if out is None:
        out = torch.empty((n, cols // 2 if swiglu else cols), dtype=a.dtype, device=a.device)
    calls["gemm_tc"] += 1
    _check(lib.tis_gemm_tc(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), out.stride(0), n, cols, k,
                           EPI_SWIGLU if swiglu else EPI_STORE, _p(tc_fault()), _stream()), lib)
    return out


#: bfloat16 library products go to cuBLAS directly (the same kernels as torch.mm, a third of the host
#: time per call); TIS_LIBRARY_GEMM=torch sends them through torch.mm instead
LIBRARY_GEMM_DIRECT = os.environ.get("TIS_LIBRARY_GEMM", "direct") != "torch"
_blas_state = None          # None: not tried yet; False: unavailable; else the workspace tensor


def _library_gemm(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], f32_out: bool) -> Optional[torch.Tensor]:
    """``a @ w`` by a direct cuBLAS call, or None when that is not possible (then torch.mm does it)."""
    global _blas_state, launches
    if not LIBRARY_GEMM_DIRECT or _blas_state is False:
        return None
    if (a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.stride(1) != 1 or w.stride(1) != 1
            or a.stride(0) < a.shape[1] or w.stride(0) < w.shape[1]):
        return None
    lib = library()
    if _blas_state is None:
        ws = torch.empty(32 << 20, dtype=torch.uint8, device=a.device)
        _blas_state = ws if lib.tis_gemm_library_init(_p(ws), ctypes.c_size_t(ws.numel())) else False
        if _blas_state is False:
            return None
    n, k = a.shape
    cols = w.shape[1]
    want = torch.float32 if f32_out else torch.bfloat16
    if out is None:
        out = torch.empty((n, cols), dtype=want, device=a.device)
    elif out.dtype != want or out.stride(1) != 1 or out.stride(0) < cols:
        return None
    calls["gemm_library"] += 1
    status = lib.tis_gemm_library(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), out.stride(0), n, cols, k,
                                  int(f32_out), _stream())
    if status != 0:
        raise KernelError(lib.tis_last_error().decode())
    return out


def gemm(a, w: torch.Tensor, out: Optional[torch.Tensor] = None, sink: Optional[ResidualSink] = None):
    """``a (n, K) @ w (K, N)`` in the dtype of ``a``; float32 means true float32.  Few bfloat16
    rows go to the weight-streaming kernel of this library, many to its tcgen05 kernel,
    everything else to the library product.

    ``a`` may be ``ScaledRows``.  With ``sink``, a product that goes to a weight-streaming kernel adds its
    result to the residual stream itself and returns ``ScaledRows`` for the norm that follows; any other
    product ignores the sink and returns its result, which the caller adds as before."""
    scaled = a if isinstance(a, ScaledRows) else None
    if scaled is not None:
        a = scaled.rows
    if a.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
        raise KernelError("float32 products must not run in TF32: torch.backends.cuda.matmul.allow_tf32 is set")
    streams = _stream_pays(a.shape[0], a.shape[1], w.shape[1]) and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
    if (_skinny_ok(a, w) and (streams or _ring_tiles(w.shape[1], a.shape[1]) <= RING_MAX_TILES)) or \
            (_skinny_ok(a, w, STREAM_MAX_ROWS) and streams):
        if sink is not None and not _sink_fits(sink, a.shape[0], w.shape[1], out):
            sink = None
        return gemm_skinny(scaled if scaled is not None else a, w, out, sink=sink)
    if _skinny_ok(a, w) and a.shape[1] >= 2 * w.shape[1] and _swap_ok(a, w, out):
        # a long share of K per CTA and a tall matrix: the tcgen05 kernel with swapped operands
        if sink is not None and not (_sink_fits(sink, a.shape[0], w.shape[1], out) and sink.values.stride(0) % 4 == 0
                                     and sink.values.data_ptr() % 16 == 0 and sink.weight.data_ptr() % 16 == 0):
            sink = None
        return gemm_swap(scaled if scaled is not None else a, w, out, sink=sink)
    if scaled is not None:
        a = scaled.dense()
    if _tc_ok(a, w, TC_PLAIN_MIN_ROWS) and (out is None or (out.stride(1) == 1 and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0)):
        return gemm_tc(a, w, out)
    direct = _library_gemm(a, w, out, False)
    if direct is not None:
        return direct
    if out is None:
        return torch.mm(a, w)
    return torch.mm(a, w, out=out)


def gemm_swiglu(a, w_gu: torch.Tensor, hidden: int, block: int) -> torch.Tensor:
    """``swiglu(a @ w_gu)``: (n, hidden).  ``w_gu`` (K, 2*hidden) holds gate and up columns in
    alternating blocks of ``block``.  Few bfloat16 rows with block 32: one kernel with the
    gating in its epilogue; else the product and the gating kernel.  ``a`` may be ``ScaledRows``."""
    scaled = a if isinstance(a, ScaledRows) else None
    if scaled is not None:
        a = scaled.rows
    if block == 32 and _skinny_ok(a, w_gu, SKINNY_SWIGLU_MAX_ROWS) and (
            _ring_tiles(w_gu.shape[1], a.shape[1]) <= RING_MAX_TILES or not _swap_ok(a, w_gu, swiglu=True)):
        return gemm_skinny(scaled if scaled is not None else a, w_gu, swiglu=True)
    if (block == 32 and _skinny_ok(a, w_gu, SWAP_SWIGLU_MAX_ROWS) and w_gu.shape[1] % 64 == 0
            and a.data_ptr() % 16 == 0 and w_gu.data_ptr() % 16 == 0):
        return gemm_swap(scaled if scaled is not None else a, w_gu, swiglu=True)
    if scaled is not None:
        a = scaled.dense()
    if block == 32 and _tc_ok(a, w_gu, TC_MIN_ROWS) and w_gu.shape[1] % 64 == 0:
        return gemm_tc(a, w_gu, swiglu=True)
    gu = gemm(a, w_gu)
    out = torch.empty((a.shape[0], hidden), dtype=a.dtype, device=a.device)
    return swiglu(gu, out, block)


def gemm_f32_out(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``a (n, K) @ w (K, N)`` with a float32 result whatever the dtype of the operands."""
    if a.dtype == torch.float32:
        return gemm(a, w)
    direct = _library_gemm(a, w, None, True)
    if direct is not None:
        return direct
    return torch.mm(a, w, out_dtype=torch.float32)


# ---------------------------------------------------------------------------------------
# row-wise kernels
# ---------------------------------------------------------------------------------------

def embed_rows(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r] = float(table[tokens[r]]); out is the float32 residual stream (n, d)."""
    lib = library()
    n, d = out.shape
    _check(lib.tis_embed_rows(_dt(table), _p(table), _p(tokens), _p(out), n, d, _stream()), lib)
    return out


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], scale: torch.Tensor, eps: float,
                out: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """residual += delta (when given), then out = residual*sqrt(d)/(||residual||+eps)*scale."""
    lib = library()
    n, d = residual.shape
    ref = out if out is not None else delta
    _check(lib.tis_add_rmsnorm(_dt(ref), _p(residual), _p(delta), _p(scale), _f(eps), _p(out), n, d, _stream()), lib)
    return out


def residual_add(residual: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    lib = library()
    n, d = residual.shape
    _check(lib.tis_residual_add(_dt(delta), _p(residual), _p(delta), n, d, _stream()), lib)
    return residual


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, row_slot: torch.Tensor, cos: torch.Tensor,
                  sin: torch.Tensor, plane: Optional[torch.Tensor], block_table: Optional[torch.Tensor],
                  num_heads: int, kv_heads: int, head_dim: int, page_size: int, fault: torch.Tensor,
                  interleaved: bool = False, write_kv: bool = True) -> None:
    """Rotate the queries of ``qkv`` (n, (H+2*KVH)*hd) in place; rotate the keys and write
    keys and values of every row into its page of ``plane`` [pages, 2, KVH, page, hd]."""
    lib = library()
    n = qkv.shape[0]
    rot = 2 * cos.shape[1]
    write = bool(write_kv and plane is not None)
    _check(lib.tis_rope_kv_write(
        _dt(qkv), _p(qkv), qkv.stride(0), _p(positions), _p(row_slot), _p(cos), _p(sin),
        _p(plane if write else None), _p(block_table if write else None),
        block_table.stride(0) if write else 0, plane.shape[0] if write else 0,
        n, num_heads, kv_heads, head_dim, rot, int(interleaved), page_size, int(write), _p(fault), _stream()), lib)


_attn_libs = {}

def attention_library(head_dim: int):
    """The tensor-core attention kernels for one head size, compiled when first needed."""
    lib = _attn_libs.get(head_dim)
    if lib is None:
        library()
        lib = ctypes.CDLL(_build.build_attention(head_dim))
        lib.tis_last_error.restype = ctypes.c_char_p
        lib.tis_attn_scratch_floats.restype = ctypes.c_size_t
        lib.resident = {}
        lib.tc_attention = bool(lib.tis_attn_tc_supported())
        if lib.tis_attn_head_dim() != head_dim:
            raise KernelError(f"attention library built for head size {lib.tis_attn_head_dim()}, wanted {head_dim}")
        _attn_libs[head_dim] = lib
    return lib


#: long prompt portions (tiles of up to 128 rows) go to the tcgen05 attention kernel where the head
#: size (64, 128) and the page size (16..128) allow it; TIS_TC_ATTENTION=0 keeps them on the
#: mma.sync kernel
TC_ATTENTION = os.environ.get("TIS_TC_ATTENTION", "1") != "0"
TC_ATTENTION_MIN_TILES = 2
TC_ATTENTION_SHORT_CONTEXT = 1024

#: CTAs of the attention kernels that are resident at a time when the library cannot be asked
#: (148 SMs, two CTAs each at head size 128)
ATTN_RESIDENT_CTAS = 148 * 2
#: cost of starting and finishing a CTA, and of merging one more split, in units of one 64-key tile
ATTN_CTA_OVERHEAD_TILES = 8.0
ATTN_MERGE_PER_SPLIT_TILES = 0.1
#: most key splits of a decode tile (one cluster): 16, a cluster size that the device allows on request, while
#: the CTAs of the kernel with a producer warp are all resident (two to an SM); else the portable 8.  Measured
#: inside the decode step of the 0.9B model at context 4096, 8 -> 16 splits: batch 1 1.003 -> 0.938 ms a step,
#: batch 2 1.022 -> 0.977, batch 4 1.080 -> 1.051; at batch 8 (384 CTAs) 16 splits cost (17.6 -> 28.4 us a launch).
#: TIS_ATTN_MAX_SPLITS overrides.
ATTN_MAX_SPLITS_KEYS = int(os.environ.get("TIS_ATTN_MAX_SPLITS", "16"))
ATTN_DECODE_RESIDENT_CTAS = 148 * 2


def plan_splits(num_tiles: int, kv_heads: int, max_kv: int, mode_keys: bool, resident: int = ATTN_RESIDENT_CTAS,
                min_kv: Optional[int] = None):
    """(keys per split, number of splits) for contexts of up to ``max_kv`` keys.

    One CTA walks the keys of one (tile, kv head, split), 64 at a time.  With few tiles the
    SMs idle unless the keys are split; with too many splits every CTA is all overhead.
    Tiles of a prompt see different numbers of keys (``min_kv`` .. ``max_kv``, causal): without
    splits the CTA of the last tile works long after the others are done.  The number of
    splits minimises an estimate of the time: CTAs that have keys at all, each costing
    overhead + its tiles, spread over the CTAs that are resident at a time, but never less
    than the longest CTA; plus the cost of merging."""
    total_tiles = max(1, (max_kv + 63) // 64)
    lo_tiles = total_tiles if min_kv is None else max(1, (min(min_kv, max_kv) + 63) // 64)
    # the splits are one thread-block cluster: at most 8 CTAs, or 16 for decode tiles (a cluster size
    # that the device allows on request)
    limit = min(total_tiles, ATTN_MAX_SPLITS_KEYS if mode_keys else 8)
    if not mode_keys and lo_tiles < 0.75 * total_tiles:
        # a prompt from its start: tiles see very different numbers of keys.  The CTAs of a cluster
        # leave together, so a split without keys would hold its place until the longest one is
        # done: splitting gains nothing there (measured: a 2048-token prompt gets slower).
        limit = 1
    best, best_cost = 1, None
    for s in range(1, limit + 1):
        per_tiles = (total_tiles + s - 1) // s
        if (total_tiles + per_tiles - 1) // per_tiles != s:
            continue
        if s > 8 and (s != 16 or num_tiles * kv_heads * s > ATTN_DECODE_RESIDENT_CTAS):
            continue                   # above the portable cluster size only 16, and only while all CTAs are resident
        # tiles with key counts spread evenly from lo_tiles to total_tiles
        work, ctas = 0.0, 0.0
        samples = min(num_tiles, 16)
        for i in range(samples):
            kv = lo_tiles + (total_tiles - lo_tiles) * (i + 0.5) / samples
            full, rest = divmod(kv, per_tiles)
            ctas += full + (1 if rest > 1e-9 else 0)
            work += full * (ATTN_CTA_OVERHEAD_TILES + per_tiles) + ((ATTN_CTA_OVERHEAD_TILES + rest) if rest > 1e-9 else 0)
        scale = num_tiles * kv_heads / samples
        ctas, work = ctas * scale, work * scale
        longest = ATTN_CTA_OVERHEAD_TILES + per_tiles
        if lo_tiles == total_tiles:
            # equal CTAs run in whole rounds: one CTA more than fit at a time costs a second round
            cost = math.ceil(ctas / resident - 1e-9) * longest
        else:
            cost = max(longest, work / min(resident, max(ctas, 1.0)))
        if s > 1:
            cost += ATTN_MERGE_PER_SPLIT_TILES * s
            if not mode_keys:
                cost += 1.0            # 64 rows of partial outputs go through shared memory of the cluster
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    per = ((total_tiles + best - 1) // best) * 64
    return per, max(1, (max_kv + per - 1) // per)


#: decode steps: the attention kernel rotates queries and keys and writes the cache itself
#: (TIS_ATTN_ROTARY=0: the rope_kv_write kernel does, in a launch of its own, as for every other step)
ATTN_ROTARY = os.environ.get("TIS_ATTN_ROTARY", "1") != "0"


def rotary_fusable(q: torch.Tensor, step, num_heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether ``paged_attention`` can take rows whose queries are not rotated yet and whose keys and
    values are not in the cache yet (``rotary=``): a decode step (one row per request) in bfloat16, a head
    size the kernel rotates in registers, at most 16 query heads per kv head."""
    return (ATTN_ROTARY and q.dtype == torch.bfloat16 and step is not None and getattr(step, "decode_only", False)
            and head_dim % 32 == 0 and kv_heads > 0 and num_heads % kv_heads == 0 and num_heads // kv_heads <= 16)


def paged_attention(q: torch.Tensor, out: torch.Tensor, plane: torch.Tensor, block_table: torch.Tensor,
                    positions: torch.Tensor, row_slot: torch.Tensor, num_heads: int, kv_heads: int,
                    head_dim: int, page_size: int, window: Optional[int], fault: torch.Tensor,
                    step=None, rotary=None, write_kv: bool = True) -> torch.Tensor:
    """Causal attention of the step's rows over the cache.  ``q`` is (n, >= H*hd) with the
    queries first in each row (row stride free); ``out`` is (n, H*hd).  The row at position
    p of slot s sees keys max(0, p-window+1)..p of ``plane`` through ``block_table[s]``.

    float32: CUDA-core kernel, everything in 32-bit.  bfloat16: tensor-core kernels over
    tiles of rows (``kernels.attention_plan``), keys of long contexts split over CTAs.

    ``rotary=(cos, sin)`` (only where ``rotary_fusable``): the rows of ``q`` are the projection's output
    as it is, [queries | keys | values]; the kernel rotates queries and keys itself (half-split pairs,
    tables [positions, hd/2] float32) and, with ``write_kv``, writes the rows' keys and values into
    their pages — what ``rope_kv_write`` does in a launch of its own everywhere else."""
    lib = library()
    n = q.shape[0]
    scale = 1.0 / math.sqrt(head_dim)
    if rotary is not None and not rotary_fusable(q, step, num_heads, kv_heads, head_dim):
        raise KernelError("paged_attention: rotary encoding inside the kernel is for decode steps in bfloat16")
    if q.dtype == torch.float32:
        _check(lib.tis_paged_attention_simt(
            _dt(q), _p(q), q.stride(0), _p(out), out.stride(0), _p(plane), _p(block_table), block_table.stride(0),
            plane.shape[0], _p(positions), _p(row_slot), n, num_heads, kv_heads, head_dim, page_size,
            int(window or 0), _f(scale), _p(fault), _stream()), lib)
        return out
    if kv_heads <= 0 or num_heads % kv_heads:
        raise KernelError(f"paged_attention: {num_heads} query heads are not a multiple of {kv_heads} kv heads")
    g = num_heads // kv_heads
    if g > 64:
        raise KernelError(f"paged_attention: {g} query heads per kv head; the bfloat16 kernels take up to 64")
    alib = attention_library(head_dim)
    min_kv = None
    from . import attention_plan
    if step is not None:
        tiles = step.plan(attention_plan.planner(g))
        max_kv = step.max_position + 1
        min_kv = getattr(step, "min_position", None)
        min_kv = None if min_kv is None else min_kv + 1
    else:
        tiles = attention_plan.infer_tiles(positions, row_slot, g)
        max_kv = int(positions.max().item()) + 1 if n else 1
    rows_tiles = tiles.rows
    w0, wn, wide_count = getattr(tiles, "wide", (None, None, 0))
    # One CTA of the tcgen05 kernel walks all keys of its 128 rows (no key splits yet).  Measured at the
    # 0.9B sizes: with two or more such tiles in the step it wins (256 rows ending at 4096: 51 against
    # 84 us), a single tile deep inside a long context is faster on the mma.sync kernel, which splits
    # the keys over a cluster (128 rows ending at 4096: 51 against 34 us; ending at 1024: a tie).
    tc_pays = wide_count >= TC_ATTENTION_MIN_TILES or max_kv <= TC_ATTENTION_SHORT_CONTEXT
    if wide_count and TC_ATTENTION and tc_pays and page_size in (16, 32, 64, 128) and alib.tc_attention:
        # long portions: the tcgen05 kernel takes them as tiles of 128 rows; the others stay below
        calls["attn_tc"] += 1
        _check(alib.tis_attn_tc(_p(q), q.stride(0), n, _p(out), out.stride(0), _p(plane), _p(block_table),
                                block_table.stride(0), plane.shape[0], _p(positions), _p(row_slot), _p(w0), _p(wn),
                                wide_count, num_heads, kv_heads, page_size, int(window or 0), _f(scale), _p(fault),
                                _stream()), alib)
        skip = tiles.rows_in_wide
        if skip == tiles.rows[2]:
            rows_tiles = (None, None, 0)
        else:
            rows_tiles = (tiles.rows[0][skip:], tiles.rows[1][skip:], tiles.rows[2] - skip)
    if rotary is not None:
        row0, rows, count = tiles.keys
        if tiles.rows[2] or wide_count or tiles.keys_max_rows != 1:
            raise KernelError("paged_attention: rotary encoding inside the kernel needs tiles of one row")
        half = int(g <= 8)
        resident = alib.resident.get((1, half))
        if resident is None:
            resident = alib.resident[(1, half)] = alib.tis_attn_resident_ctas(1, half)
        per, splits = plan_splits(count, kv_heads, max_kv, True, resident, None)
        calls["attn_keys_rotary"] += 1
        cos, sin = rotary
        if getattr(tiles, "keys_identity", False) and count == n:
            row0 = rows = None          # tile i is row i: the kernel reads no tile arrays
        _check(alib.tis_attn_decode_rope(_p(q), q.stride(0), _p(out), out.stride(0), _p(plane), _p(block_table),
                                         block_table.stride(0), plane.shape[0], _p(positions), _p(row_slot), _p(row0),
                                         _p(rows), count, n, num_heads, kv_heads, page_size, int(window or 0),
                                         _f(scale), per, splits, _p(cos), _p(sin), int(bool(write_kv)), _p(fault),
                                         _stream()), alib)
        return out
    for mode, (row0, rows, count) in ((1, tiles.keys), (0, rows_tiles)):
        if count == 0:
            continue
        max_rows = tiles.keys_max_rows if mode == 1 else 0
        half = int(mode == 1 and 0 < max_rows * g <= 8)
        resident = alib.resident.get((mode, half))
        if resident is None:
            resident = alib.resident[(mode, half)] = alib.tis_attn_resident_ctas(mode, half)
        per, splits = plan_splits(count, kv_heads, max_kv, mode == 1, resident, None if mode == 1 else min_kv)
        calls["attn_keys" if mode == 1 else "attn_rows"] += 1
        # at most eight splits (plan_splits): they merge inside a thread-block cluster, without scratch
        _check(alib.tis_attn_mma(mode, _p(q), q.stride(0), _p(out), out.stride(0), _p(plane), _p(block_table),
                                 block_table.stride(0), plane.shape[0], _p(positions), _p(row_slot), _p(row0),
                                 _p(rows), count, max_rows, n, num_heads, kv_heads, page_size, int(window or 0), _f(scale),
                                 per, splits, _p(None), _p(fault), _stream()), alib)
    return out


def swiglu(gu: torch.Tensor, out: torch.Tensor, block: Optional[int] = None) -> torch.Tensor:
    """out[r, j] = silu(gate_j) * up_j where a row of ``gu`` holds gate and up columns in
    alternating blocks of ``block`` (default: the hidden size, i.e. [all gates | all ups])."""
    lib = library()
    n, f = out.shape
    _check(lib.tis_swiglu(_dt(gu), _p(gu), _p(out), n, f, block or f, _stream()), lib)
    return out


def mtp_input(h_prev: torch.Tensor, state: torch.Tensor, row_slot: torch.Tensor, row_last: torch.Tensor,
              tokens: torch.Tensor, table: torch.Tensor, scale: torch.Tensor, eps: float,
              out: torch.Tensor) -> torch.Tensor:
    """out[r] = [h_prev of the row before r (the slot's saved row for a request's first row) |
    rmsnorm(table[tokens[r]])]; saves h_prev[row_last[r]] into the slot for the next step."""
    lib = library()
    n, d = h_prev.shape
    _check(lib.tis_mtp_input(_dt(h_prev), _p(h_prev), _p(state), _p(row_slot), _p(row_last), _p(tokens),
                             _p(table), _p(scale), _f(eps), _p(out), n, d, _stream()), lib)
    return out


# ---------------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------------

def sample_rows(logits: torch.Tensor, temps: torch.Tensor, top_ks: torch.Tensor, top_ps: torch.Tensor,
                penalties: torch.Tensor, slots: Optional[torch.Tensor], seen_bitmap: Optional[torch.Tensor],
                seeds: torch.Tensor, counters: torch.Tensor, out_tokens: torch.Tensor,
                probs_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 ``logits`` (k, V); see csrc/sampling.cu for the order of
    the transformations.  ``seen_bitmap`` (slots, ceil(V/32)) int32 gets the drawn token's bit."""
    lib = library()
    k, v = logits.shape
    words = seen_bitmap.shape[1] if seen_bitmap is not None else 0
    _check(lib.tis_sample_rows(_p(logits), k, v, _p(temps), _p(top_ks), _p(top_ps), _p(penalties), _p(slots),
                               _p(seen_bitmap), words, _p(seeds), _p(counters), _p(out_tokens), _p(probs_out),
                               _stream()), lib)
    return out_tokens


def sample_stage_limit(entries: int) -> None:
    """For tests: the most entries of a row that a CTA of the sampling kernel keeps in shared memory (fewer
    means more CTAs a row; 0: none, every pass reads the logits; -1: what the device allows)."""
    _check(library().tis_sample_stage_limit(int(entries)), library())


def bitmap_set(bitmap_row: torch.Tensor, tokens: torch.Tensor) -> None:
    lib = library()
    _check(lib.tis_bitmap_set(_p(bitmap_row), _p(tokens), tokens.numel(), _stream()), lib)
