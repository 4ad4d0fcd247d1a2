"""Plan objects: the host-built segment schedule of one varlen problem, uploaded
once and reused by every call on the same lists.

A plan is what replaces the per-call host work of the upstream launchers
(``csrc/cuda/spBlkGEMM.cu:943-1006``: seven device->host syncs, a host loop over
tiles and an upload per GEMM call; ``csrc/cuda/spBlkSoftmax.cu:358-396``: a
per-row table).  Lists are taken on the host; running a plan launches kernels
on torch's current stream and does not synchronise.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib as L

_DTYPES = {torch.float16: L.BLK_F16, torch.bfloat16: L.BLK_BF16, torch.float32: L.BLK_F32}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise RuntimeError(f"blockedattention_b200: dtype {dt} is not supported (float16, bfloat16, float32)")


def _host_i64(x) -> Optional[np.ndarray]:
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        x = x.detach().to("cpu", torch.int64).numpy()
    return np.ascontiguousarray(np.asarray(x, dtype=np.int64))


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _rec(*fields):
    return np.dtype([tuple(f) for f in fields])


_TILE_ITEM = _rec(("seg", "<i4"), ("tm", "<i4"), ("tn", "<i4"), ("ntn", "<i4"))
_SMALL_ITEM = _rec(("offA", "<i8"), ("offB", "<i8"), ("offC", "<i8"), ("M", "<i4"), ("N", "<i4"))
_VIEW = _rec(("K", "<i8"), ("residue", "<i8"))
# name -> (blk_table_t value, record layout): mirrors of the schedule records of csrc/blk_internal.h
TABLES = {
    "segments": (0, _rec(("offA", "<i8"), ("offB", "<i8"), ("offC", "<i8"), ("M", "<i4"), ("N", "<i4"), ("K", "<i4"),
                         ("clsIn", "u1"), ("clsOut", "u1"), ("pad", "u1", (2,)))),
    "tile_items": (1, _TILE_ITEM),
    "simt_items": (2, _TILE_ITEM),
    "small_items_32": (3, _SMALL_ITEM),
    "small_items_64": (4, _SMALL_ITEM),
    "umma_items": (5, _rec(("views", "<i4"), ("tm", "<i4"), ("rowA", "<i4"), ("rowB", "<i4"), ("offC", "<i8"),
                           ("M", "<i4"), ("N", "<i4"), ("K", "<i4"), ("ch0", "<i4"), ("nch", "<i4"), ("pad", "<i4"))),
    "pv_items": (6, _rec(("offA", "<i8"), ("offC", "<i8"), ("rowB", "<i4"), ("M", "<i4"), ("K", "<i4"), ("pad", "<i4"))),
    "packs": (7, _rec(("offA", "<i8"), ("offB", "<i8"), ("rowsA", "<i4"), ("rowsB", "<i4"), ("first_block", "<i4"),
                      ("nblocks", "<i4"))),
    "pack_blocks": (8, _rec(("offC", "<i8"), ("rowA", "<i4"), ("rowB", "<i4"), ("M", "<i4"), ("N", "<i4"),
                            ("nblocks", "<i4"), ("pad", "<i4"))),
    "softmax_chunks": (9, _rec(("off", "<i8"), ("rows", "<i4"), ("cols", "<i4"))),
    "softmax_windows": (10, _rec(("off", "<i8"), ("nbytes", "<i4"), ("first_piece", "<i4"), ("npieces", "<i4"),
                                 ("pad", "<i4"))),
    "flash_items": (11, _rec(("rowQ", "<i4"), ("rowKV", "<i4"), ("M", "<i4"), ("N", "<i4"))),
    "umma_views_a": (12, _VIEW),
    "umma_views_b": (13, _VIEW),
}


class _Plan:
    def __init__(self):
        self._h = C.c_void_p()

    def close(self):
        if getattr(self, "_h", None) is not None and self._h:
            L.lib.blk_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def extents(self):
        a, b, c = C.c_int64(), C.c_int64(), C.c_int64()
        L.check(L.lib.blk_plan_extents(self._h, C.byref(a), C.byref(b), C.byref(c)))
        return a.value, b.value, c.value

    @property
    def summary(self) -> dict:
        arr = (C.c_int64 * 8)()
        L.check(L.lib.blk_plan_summary(self._h, arr))
        keys = ["segments", "small_items", "tile_items", "umma_items", "softmax_chunks", "launches", "simt_items", "packs"]
        return {k: int(arr[i]) for i, k in enumerate(keys)}

    def table(self, name: str) -> np.ndarray:
        """One of the schedule's tables as a numpy record array (a copy), for tests and debugging; ``name`` is a key
        of ``TABLES``.  The record layouts are the library's own and follow its version."""
        which, dtype = TABLES[name]
        n, rec = C.c_int64(), C.c_int64()
        L.check(L.lib.blk_plan_table(self._h, which, None, 0, C.byref(n), C.byref(rec)))
        if rec.value != dtype.itemsize:
            raise RuntimeError(f"table {name}: the library's records have {rec.value} bytes, this module expects "
                               f"{dtype.itemsize}")
        out = np.empty(n.value // dtype.itemsize, dtype)
        if n.value:
            L.check(L.lib.blk_plan_table(self._h, which, out.ctypes.data_as(C.c_void_p), n.value, C.byref(n), None))
        return out

    @property
    def work(self):
        """(algorithmic flops, algorithmic bytes) of one run over all heads."""
        f, b = C.c_double(), C.c_double()
        L.check(L.lib.blk_plan_work(self._h, C.byref(f), C.byref(b)))
        return f.value, b.value

    def check(self):
        """Synchronises the current stream and raises if a kernel reported a timed-out wait."""
        L.check(L.lib.blk_plan_check(self._h, C.c_void_p(_stream_ptr(self.device))))

    def _ran(self):
        # A kernel whose bounded wait gives up only sets the plan's status word and returns with its output
        # incomplete; nothing reads that word unless asked.  BLK_CHECK=1 asks after every run (one stream
        # synchronisation per call: a debugging switch, not a production setting).
        if os.environ.get("BLK_CHECK", "0") not in ("", "0"):
            self.check()


class GemmPlan(_Plan):
    """Schedule for ``out_s = epilogue(scale * A_s B_s^T)`` over S segments and H heads.

    ``MList/NList/KList``: host sequences (or tensors, copied to the host once).
    ``accum``: optional ``(mat1Accum, mat2Accum, outAccum)`` triple; default is
    the packed offsets ``cumsum([0, M*K])`` etc. (upstream
    ``csrc/sparseBlockedAttention.cpp:22-29``).  ``device=None`` builds the
    schedule only (no GPU needed).
    """

    def __init__(self, MList, NList, KList, H: int, dtype_in: torch.dtype, dtype_out: Optional[torch.dtype] = None,
                 transpose1: bool = False, transpose2: bool = False, softmax: bool = False,
                 accum: Optional[Sequence] = None, device=None):
        super().__init__()
        self.M, self.N, self.K = _host_i64(MList), _host_i64(NList), _host_i64(KList)
        if not (len(self.M) == len(self.N) == len(self.K)):
            raise RuntimeError("MList, NList and KList must have the same length")
        self.S, self.H = len(self.M), int(H)
        self.dtype_in = dtype_in
        self.dtype_out = dtype_out if dtype_out is not None else dtype_in
        self.softmax = bool(softmax)
        self.ta, self.tb = bool(transpose1), bool(transpose2)
        self.device = torch.device(device) if device is not None else None
        a1 = a2 = ao = None
        if accum is not None:
            a1, a2, ao = (_host_i64(a) for a in accum)
            for a in (a1, a2, ao):
                if len(a) != self.S + 1:
                    raise RuntimeError("offset arrays must have one more entry than the lists")
        dev = -1 if self.device is None else (self.device.index if self.device.index is not None
                                               else torch.cuda.current_device())
        L.check(L.lib.blk_gemm_plan_create(
            C.byref(self._h), L.i64(self.M), L.i64(self.N), L.i64(self.K), L.i64(a1), L.i64(a2), L.i64(ao),
            self.S, self.H, dtype_code(self.dtype_in), dtype_code(self.dtype_out), int(transpose1), int(transpose2),
            L.BLK_EPI_SOFTMAX if softmax else L.BLK_EPI_SCORES, dev))
        self.Dm1, self.Dm2, self.Dout = self.extents

    @property
    def offsets(self):
        a1 = np.empty(self.S + 1, np.int64); a2 = np.empty_like(a1); ao = np.empty_like(a1)
        L.check(L.lib.blk_plan_offsets(self._h, L.i64(a1), L.i64(a2), L.i64(ao)))
        return a1, a2, ao

    def run(self, mat1: torch.Tensor, mat2: torch.Tensor, out: Optional[torch.Tensor] = None,
            scale: float = 1.0) -> torch.Tensor:
        if self.device is None:
            raise RuntimeError("this plan was built without a device")
        for name, t, D in (("mat1", mat1, self.Dm1), ("mat2", mat2, self.Dm2)):
            if not t.is_cuda:
                raise RuntimeError(f"{name} must be a CUDA tensor")
            if not t.is_contiguous():
                raise RuntimeError(f"{name} must be contiguous")
            if t.dtype != self.dtype_in:
                raise RuntimeError(f"{name} has dtype {t.dtype}, the plan was built for {self.dtype_in}")
            if t.numel() != self.H * D:
                raise RuntimeError(f"{name} has {t.numel()} elements, expected H*D = {self.H}*{D}")
        if out is None:
            out = torch.empty((self.H, self.Dout), dtype=self.dtype_out, device=mat1.device)
        elif (not out.is_cuda or not out.is_contiguous() or out.dtype != self.dtype_out
              or out.numel() != self.H * self.Dout):
            raise RuntimeError("out must be a contiguous CUDA tensor of the plan's dtype with H*Dout elements")
        if mat1.data_ptr() % 16:
            mat1 = mat1.clone()
        if mat2.data_ptr() % 16:
            mat2 = mat2.clone()
        if out.data_ptr() % 16:
            raise RuntimeError("out must be 16-byte aligned")
        with torch.cuda.device(mat1.device):
            L.check(L.lib.blk_gemm_run(self._h, C.c_void_p(mat1.data_ptr()), C.c_void_p(mat2.data_ptr()),
                                       C.c_void_p(out.data_ptr()), C.c_float(scale),
                                       C.c_void_p(_stream_ptr(mat1.device))))
        self._ran()
        return out


    def run_token_major(self, mat1: torch.Tensor, mat2: torch.Tensor, out: Optional[torch.Tensor] = None,
                        scale: float = 1.0) -> torch.Tensor:
        """Same as :meth:`run` for token-major operands ``mat1 -> (sum m_s, H, d)``, ``mat2 -> (sum n_s, H, d)``
        (the rows of all segments in batch order); the result is the packed head-major ``(H, Dout)`` buffer.
        Needs a batch the tensor-map kernels take whole: 16-bit, one ``K = d`` that is a multiple of 8."""
        if self.device is None:
            raise RuntimeError("this plan was built without a device")
        d = int(self.K[0]) if self.S else 0
        for name, t, rows in (("mat1", mat1, int(self.M.sum())), ("mat2", mat2, int(self.N.sum()))):
            if not t.is_cuda or not t.is_contiguous() or t.dtype != self.dtype_in:
                raise RuntimeError(f"{name} must be a contiguous CUDA tensor of the plan's dtype")
            if t.dim() != 3 or tuple(t.shape) != (rows, self.H, d):
                raise RuntimeError(f"{name} must have shape (rows, H, d) = ({rows}, {self.H}, {d}), got {tuple(t.shape)}")
            if t.data_ptr() % 16:
                raise RuntimeError(f"{name} must be 16-byte aligned")
        if out is None:
            out = torch.empty((self.H, self.Dout), dtype=self.dtype_out, device=mat1.device)
        elif (not out.is_cuda or not out.is_contiguous() or out.dtype != self.dtype_out
              or out.numel() != self.H * self.Dout or out.data_ptr() % 16):
            raise RuntimeError("out must be a contiguous, 16-byte aligned CUDA tensor of the plan's dtype with H*Dout elements")
        with torch.cuda.device(mat1.device):
            L.check(L.lib.blk_gemm_run_strided(self._h, C.c_void_p(mat1.data_ptr()), self.H * d, d,
                                               C.c_void_p(mat2.data_ptr()), self.H * d, d,
                                               C.c_void_p(out.data_ptr()), C.c_float(scale),
                                               C.c_void_p(_stream_ptr(mat1.device))))
        self._ran()
        return out


class AttentionPlan(_Plan):
    """Fused ``softmax(scale * Q_s K_s^T) V_s``, head dimension ``d`` 64 or 128, fp16 or bf16.  A batch whose every
    segment has at most 64 query and 64 key rows (``d = 64``) runs on the pack kernel, any other on the tcgen05
    attention kernel; ``small_only=True`` asks for the pack kernel or ``RuntimeError`` (BLK_ERR_UNSUPPORTED)."""

    def __init__(self, MList, NList, H: int, dtype: torch.dtype, device=None, d: int = 64, small_only: bool = False):
        super().__init__()
        self.M, self.N = _host_i64(MList), _host_i64(NList)
        if len(self.M) != len(self.N):
            raise RuntimeError("MList and NList must have the same length")
        self.S, self.H, self.dtype = len(self.M), int(H), dtype
        self.device = torch.device(device) if device is not None else None
        dev = -1 if self.device is None else (self.device.index if self.device.index is not None
                                               else torch.cuda.current_device())
        self.d = int(d)
        if small_only:
            if self.d != 64:
                raise RuntimeError("the pack kernel needs head dimension 64")
            L.check(L.lib.blk_attention_plan_create(C.byref(self._h), L.i64(self.M), L.i64(self.N), self.S, self.H,
                                                    dtype_code(dtype), dev))
        else:
            L.check(L.lib.blk_attention_plan_create_dim(C.byref(self._h), L.i64(self.M), L.i64(self.N), self.S, self.H,
                                                        self.d, dtype_code(dtype), dev))
        self.Dq, self.Dkv = int(self.M.sum()) * self.d, int(self.N.sum()) * self.d

    def run(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None,
            scale: float = 1.0) -> torch.Tensor:
        if self.device is None:
            raise RuntimeError("this plan was built without a device")
        for name, t, D in (("q", q, self.Dq), ("k", k, self.Dkv), ("v", v, self.Dkv)):
            if not t.is_cuda or not t.is_contiguous() or t.dtype != self.dtype or t.numel() != self.H * D:
                raise RuntimeError(f"{name} must be a contiguous CUDA tensor of the plan's dtype with H*{D} elements")
        if out is None:
            out = torch.empty((self.H, self.Dq), dtype=self.dtype, device=q.device)
        elif not out.is_cuda or not out.is_contiguous() or out.dtype != self.dtype or out.numel() != self.H * self.Dq:
            raise RuntimeError("out must be a contiguous CUDA tensor of the plan's dtype with H*sum(M)*d elements")
        q, k, v = (t if t.data_ptr() % 16 == 0 else t.clone() for t in (q, k, v))
        if out.data_ptr() % 16:
            raise RuntimeError("out must be 16-byte aligned")
        with torch.cuda.device(q.device):
            L.check(L.lib.blk_attention_run(self._h, C.c_void_p(q.data_ptr()), C.c_void_p(k.data_ptr()),
                                            C.c_void_p(v.data_ptr()), C.c_void_p(out.data_ptr()), C.c_float(scale),
                                            C.c_void_p(_stream_ptr(q.device))))
        self._ran()
        return out


    def run_token_major(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None,
                        scale: float = 1.0) -> torch.Tensor:
        """Same for token-major tensors ``q, out -> (sum m_s, H, d)``, ``k, v -> (sum n_s, H, d)``, read and written
        in place through strided tensor maps (needs ``sum m_s == sum n_s`` only in so far as all four share strides)."""
        if self.device is None:
            raise RuntimeError("this plan was built without a device")
        rq, rkv = int(self.M.sum()), int(self.N.sum())
        for name, t, rows in (("q", q, rq), ("k", k, rkv), ("v", v, rkv)):
            if (not t.is_cuda or not t.is_contiguous() or t.dtype != self.dtype
                    or tuple(t.shape) != (rows, self.H, self.d) or t.data_ptr() % 16):
                raise RuntimeError(f"{name} must be a contiguous, 16-byte aligned CUDA tensor of shape "
                                   f"({rows}, {self.H}, {self.d})")
        if out is None:
            out = torch.empty((rq, self.H, self.d), dtype=self.dtype, device=q.device)
        elif (not out.is_cuda or not out.is_contiguous() or out.dtype != self.dtype
              or tuple(out.shape) != (rq, self.H, self.d) or out.data_ptr() % 16):
            raise RuntimeError(f"out must be a contiguous, 16-byte aligned CUDA tensor of shape ({rq}, {self.H}, {self.d})")
        with torch.cuda.device(q.device):
            L.check(L.lib.blk_attention_run_strided(self._h, C.c_void_p(q.data_ptr()), C.c_void_p(k.data_ptr()),
                                                    C.c_void_p(v.data_ptr()), C.c_void_p(out.data_ptr()),
                                                    self.H * self.d, self.d, C.c_float(scale),
                                                    C.c_void_p(_stream_ptr(q.device))))
        self._ran()
        return out


class SoftmaxPlan(_Plan):
    """Schedule for the row softmax of S packed (rows_s, cols_s) blocks per head."""

    def __init__(self, rowList, colList, H: int, dtype: torch.dtype, accum=None, device=None):
        super().__init__()
        self.rows, self.cols = _host_i64(rowList), _host_i64(colList)
        if len(self.rows) != len(self.cols):
            raise RuntimeError("rowList and colList must have the same length")
        self.S, self.H, self.dtype = len(self.rows), int(H), dtype
        self.device = torch.device(device) if device is not None else None
        acc = _host_i64(accum)
        if acc is not None and len(acc) != self.S + 1:
            raise RuntimeError("srcAccum must have one more entry than the lists")
        dev = -1 if self.device is None else (self.device.index if self.device.index is not None
                                               else torch.cuda.current_device())
        L.check(L.lib.blk_softmax_plan_create(C.byref(self._h), L.i64(self.rows), L.i64(self.cols), L.i64(acc),
                                              self.S, self.H, dtype_code(dtype), dev))
        self.D = self.extents[0]

    @property
    def offsets(self):
        a = np.empty(self.S + 1, np.int64)
        L.check(L.lib.blk_plan_offsets(self._h, L.i64(a), None, None))
        return a

    def run(self, src: torch.Tensor, out: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
        if self.device is None:
            raise RuntimeError("this plan was built without a device")
        if not src.is_cuda:
            raise RuntimeError("src must be a CUDA tensor")
        if not src.is_contiguous():
            raise RuntimeError("src must be contiguous")
        if src.dtype != self.dtype:
            raise RuntimeError(f"src has dtype {src.dtype}, the plan was built for {self.dtype}")
        if src.numel() != self.H * self.D:
            raise RuntimeError(f"src has {src.numel()} elements, expected H*D = {self.H}*{self.D}")
        if out is None:
            out = torch.empty((self.H, self.D), dtype=self.dtype, device=src.device)
        elif not out.is_cuda or not out.is_contiguous() or out.dtype != self.dtype or out.numel() != src.numel():
            raise RuntimeError("out must be a contiguous CUDA tensor shaped like src")
        if src.data_ptr() % 16:
            src = src.clone()
        if out.data_ptr() % 16:
            raise RuntimeError("out must be 16-byte aligned")
        with torch.cuda.device(src.device):
            L.check(L.lib.blk_softmax_run(self._h, C.c_void_p(src.data_ptr()), C.c_void_p(out.data_ptr()),
                                          C.c_float(scale), C.c_void_p(_stream_ptr(src.device))))
        self._ran()
        return out

    def run_backward(self, out: torch.Tensor, grad_out: torch.Tensor, grad_src: Optional[torch.Tensor] = None,
                     scale: float = 1.0) -> torch.Tensor:
        """``grad_src = scale * (grad_out - rowsum(out * grad_out)) * out`` for the forward result ``out`` of
        ``run(src, scale=scale)`` (upstream ``sparseBlockedSoftmaxBackwardLaunch``, csrc/cuda/spBlkSoftmax.cu:418-459)."""
        if self.device is None:
            raise RuntimeError("this plan was built without a device")
        for name, t in (("out", out), ("grad_out", grad_out)):
            if not t.is_cuda or not t.is_contiguous() or t.dtype != self.dtype or t.numel() != self.H * self.D:
                raise RuntimeError(f"{name} must be a contiguous CUDA tensor of the plan's dtype with H*D elements")
        if grad_src is None:
            grad_src = torch.empty((self.H, self.D), dtype=self.dtype, device=out.device)
        elif (not grad_src.is_cuda or not grad_src.is_contiguous() or grad_src.dtype != self.dtype
              or grad_src.numel() != out.numel()):
            raise RuntimeError("grad_src must be a contiguous CUDA tensor shaped like out")
        if out.data_ptr() % 16:
            out = out.clone()
        if grad_out.data_ptr() % 16:
            grad_out = grad_out.clone()
        if grad_src.data_ptr() % 16:
            raise RuntimeError("grad_src must be 16-byte aligned")
        with torch.cuda.device(out.device):
            L.check(L.lib.blk_softmax_backward_run(self._h, C.c_void_p(out.data_ptr()), C.c_void_p(grad_out.data_ptr()),
                                                   C.c_void_p(grad_src.data_ptr()), C.c_float(scale),
                                                   C.c_void_p(_stream_ptr(out.device))))
        self._ran()
        return grad_src
