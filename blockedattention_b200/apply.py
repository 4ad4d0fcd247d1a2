"""Python surface: ``blockGEMM`` and ``blockSoftmax`` with the upstream
signatures (``blockedAttention/apply.py:6-11`` and ``:27-30``), plus the fused
``blockAttnScores``.

Differences from upstream, all at the boundary:

* keyword-only extensions ``scale``, ``out_dtype`` and ``softmax`` (defaults
  reproduce upstream behaviour: no scale, output dtype = input dtype, separate
  softmax call);
* lists/offsets are read to the host once per distinct list tensor (kept
  alive while remembered, so an address cannot come back with other values)
  and the plan is cached under the list *values*, where upstream synchronises
  seven to eleven times per call;
* the shape checks upstream leaves to ``assert`` raise ``RuntimeError``;
* ``blockSoftmax`` passes its arguments by name, so ``srcAccum`` reaches the
  offsets parameter (upstream ``apply.py:41`` hands it to ``rowList``);
* autograd: both operators record the same backward as upstream
  (``csrc/sparseBlockedAttention.cpp:52-72``: two blocked GEMMs with permuted
  lists, offsets and transposition flags; ``:103-114``: the softmax backward
  kernel); the fused ``blockAttnScores`` chains the two.  As upstream, the
  operand gradients are laid out (m, k) / (n, k) row-major whatever the
  forward transposition flags were.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Optional

import numpy as np
import torch

from . import _lib as L
from .plan import AttentionPlan, GemmPlan, SoftmaxPlan, _host_i64

_CACHE: "OrderedDict[tuple, object]" = OrderedDict()
_CACHE_MAX = 32
# List tensors already read to the host: (data_ptr, _version, numel, dtype, device) -> (the tensor, its values as
# bytes).  The entry keeps the tensor alive, so its storage cannot be freed and handed to a tensor with other
# values while the entry exists; an in-place write moves _version.  A hit therefore costs no device->host copy,
# and the plan cache below is keyed on the values themselves, never on addresses.
_LISTS: "OrderedDict[tuple, tuple]" = OrderedDict()
_LISTS_MAX = 256


def _key_of(x):
    """Cache key of a list / offset argument: its int64 values."""
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        fast = (x.data_ptr(), x._version, x.numel(), x.dtype, str(x.device))
        hit = _LISTS.get(fast)
        if hit is not None:
            _LISTS.move_to_end(fast)
            return ("v", hit[1])
        data = _host_i64(x).tobytes()
        _LISTS[fast] = (x, data)
        while len(_LISTS) > _LISTS_MAX:
            _LISTS.popitem(last=False)
        return ("v", data)
    return ("v", np.ascontiguousarray(np.asarray(x, dtype=np.int64)).tobytes())


def _cached(key, build):
    plan = _CACHE.get(key)
    if plan is None:
        plan = build()
        _CACHE[key] = plan
        # An evicted plan is only dropped from the table: an autograd context or a queued host-pipe step may
        # still hold it, and the library handle is released when the last reference goes away.
        while len(_CACHE) > _CACHE_MAX:
            _CACHE.popitem(last=False)
    else:
        _CACHE.move_to_end(key)
    return plan


def clear_plan_cache() -> None:
    """Forgets every cached plan and list (plans still referenced elsewhere stay usable)."""
    _CACHE.clear()
    _LISTS.clear()


def check_plans() -> None:
    """Synchronises the current stream of every cached plan's device and raises ``BlkError``
    (``BLK_ERR_TIMEOUT``) if a kernel of one of them gave up a bounded device-side wait since the last check --
    the result of that call is then incomplete.  ``BLK_CHECK=1`` in the environment does this after every run."""
    for plan in list(_CACHE.values()):
        inner = getattr(plan, "plan", plan)   # a host pipe wraps its plan
        if getattr(inner, "device", None) is not None:
            inner.check()


def _check_operand(name: str, t: torch.Tensor) -> None:
    # the two TORCH_CHECKs of upstream csrc/sparseBlockedAttention.h:6-8
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be CUDA Tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous Tensor")


def _lists_from_offsets(a1, a2, ao):
    a1, a2, ao = _host_i64(a1), _host_i64(a2), _host_i64(ao)
    S = len(a1) - 1
    M = np.empty(S, np.int64); N = np.empty(S, np.int64); K = np.empty(S, np.int64)
    L.check(L.lib.blk_lists_from_offsets(L.i64(a1), L.i64(a2), L.i64(ao), S, L.i64(M), L.i64(N), L.i64(K)))
    return M, N, K


def _gemm_backward(ctx_meta, mat1, mat2, grad_out, scale):
    """The two launches of upstream sparseBlockedGEMM::backward (csrc/sparseBlockedAttention.cpp:52-72):
    mat1Grad = blockedGEMM(outGrad, mat2; offsets (out, mat2, mat1); lists (M, K, N); false, !transpose2) and
    mat2Grad = blockedGEMM(outGrad, mat1; offsets (out, mat1, mat2); lists (N, K, M); true, !transpose1)."""
    M, N, K, a1, a2, ao, ta, tb, H = ctx_meta
    g = grad_out.contiguous()
    m1 = mat1.to(g.dtype)
    m2 = mat2.to(g.dtype)
    dev = g.device
    k1 = ("gemm_bwd1", M.tobytes(), N.tobytes(), K.tobytes(), a1.tobytes(), a2.tobytes(), ao.tobytes(), tb, H, g.dtype, str(dev))
    p1 = _cached(k1, lambda: GemmPlan(M, K, N, H, g.dtype, g.dtype, False, not tb, False, accum=(ao, a2, a1), device=dev))
    k2 = ("gemm_bwd2", M.tobytes(), N.tobytes(), K.tobytes(), a1.tobytes(), a2.tobytes(), ao.tobytes(), ta, H, g.dtype, str(dev))
    p2 = _cached(k2, lambda: GemmPlan(N, K, M, H, g.dtype, g.dtype, True, not ta, False, accum=(ao, a1, a2), device=dev))
    return p1.run(g, m2, scale=scale), p2.run(g, m1, scale=scale)


class _BlockGEMMFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, mat1, mat2, plan, scale, softmax):
        out = plan.run(mat1, mat2, scale=scale)
        a1, a2, ao = plan.offsets
        ctx.meta = (plan.M, plan.N, plan.K, a1, a2, ao, plan.ta, plan.tb, plan.H)
        ctx.scale, ctx.softmax = scale, softmax
        ctx.lead = (mat1.shape, mat2.shape)
        ctx.save_for_backward(mat1, mat2, out if softmax else None)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        mat1, mat2, probs = ctx.saved_tensors
        M, N, K, a1, a2, ao, ta, tb, H = ctx.meta
        g = grad_out.contiguous()
        if ctx.softmax:
            # d(scores * scale) from d(probabilities), then the GEMM backward carries the scale
            key = ("smx_bwd_of_gemm", M.tobytes(), N.tobytes(), ao.tobytes(), H, g.dtype, str(g.device))
            sp = _cached(key, lambda: SoftmaxPlan(M, N, H, g.dtype, accum=ao, device=g.device))
            g = sp.run_backward(probs.to(g.dtype), g)
        g1, g2 = _gemm_backward(ctx.meta, mat1, mat2, g, ctx.scale)
        return g1.reshape(ctx.lead[0]).to(mat1.dtype), g2.reshape(ctx.lead[1]).to(mat2.dtype), None, None, None


class _BlockSoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, src, plan, scale):
        out = plan.run(src, scale=scale)
        ctx.plan, ctx.scale = plan, scale
        ctx.lead = src.shape
        ctx.save_for_backward(out)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (out,) = ctx.saved_tensors
        g = grad_out.contiguous()
        plan = ctx.plan
        if g.dtype != plan.dtype:  # upstream converts the saved result to the gradient's dtype
            key = ("smx_bwd_cast", plan.rows.tobytes(), plan.cols.tobytes(), plan.offsets.tobytes(), plan.H, g.dtype,
                   str(g.device))
            plan = _cached(key, lambda: SoftmaxPlan(ctx.plan.rows, ctx.plan.cols, ctx.plan.H, g.dtype,
                                                    accum=ctx.plan.offsets, device=g.device))
        return plan.run_backward(out.to(g.dtype), g, scale=ctx.scale).reshape(ctx.lead), None, None


def blockGEMM(mat1: torch.Tensor, mat2: torch.Tensor,
              mat1Accum: Optional[torch.Tensor] = None, mat2Accum: Optional[torch.Tensor] = None,
              outAccum: Optional[torch.Tensor] = None,
              MList: Optional[torch.Tensor] = None, NList: Optional[torch.Tensor] = None,
              KList: Optional[torch.Tensor] = None,
              transpose1: Optional[bool] = False, transpose2: Optional[bool] = False,
              *, scale: float = 1.0, out_dtype: Optional[torch.dtype] = None,
              softmax: bool = False) -> torch.Tensor:
    """Varlen blocked GEMM over a packed, head-major batch.

    ``mat1 -> (H, sum m_s*k_s)``, ``mat2 -> (H, sum n_s*k_s)``, result
    ``(H, sum m_s*n_s)`` with ``out_s = mat1_s @ mat2_s^T``.  Give either the
    three offset tensors (``mat1Accum = (0, m1*k1, m1*k1+m2*k2, ...)`` and so
    on) or the three lists (``MList = (m1, m2, ...)``), or both.
    ``transpose1``: mat1_s is stored (k, m); ``transpose2``: mat2_s is stored
    (k, n).  Any leading shape of mat1 flattens to H.
    """
    _check_operand("mat1", mat1)
    _check_operand("mat2", mat2)
    have_acc = mat1Accum is not None and mat2Accum is not None and outAccum is not None
    have_lists = MList is not None and NList is not None and KList is not None
    if not (have_acc or have_lists):
        raise RuntimeError("blockGEMM needs either mat1Accum/mat2Accum/outAccum or MList/NList/KList")
    if mat1.dtype != mat2.dtype:
        raise RuntimeError("mat1 and mat2 must have the same dtype")
    odt = out_dtype if out_dtype is not None else mat1.dtype
    key = ("gemm", _key_of(mat1Accum) if have_acc else None, _key_of(mat2Accum) if have_acc else None,
           _key_of(outAccum) if have_acc else None, _key_of(MList) if have_lists else None,
           _key_of(NList) if have_lists else None, _key_of(KList) if have_lists else None,
           mat1.numel(), mat1.dtype, odt, bool(transpose1), bool(transpose2), bool(softmax), str(mat1.device))

    def build():
        if have_lists:
            M, N, K = _host_i64(MList), _host_i64(NList), _host_i64(KList)
        else:
            M, N, K = _lists_from_offsets(mat1Accum, mat2Accum, outAccum)
        accum = (mat1Accum, mat2Accum, outAccum) if have_acc else None
        Dm1 = int(_host_i64(mat1Accum)[-1]) if have_acc else int((M * K).sum())
        if Dm1 <= 0 or mat1.numel() % Dm1:
            raise RuntimeError(f"mat1 has {mat1.numel()} elements, not a multiple of the packed extent {Dm1}")
        H = mat1.numel() // Dm1
        return GemmPlan(M, N, K, H, mat1.dtype, odt, bool(transpose1), bool(transpose2), bool(softmax),
                        accum=accum, device=mat1.device)

    plan = _cached(key, build)
    if mat1.shape[-1] != plan.Dm1 and mat1.numel() != plan.H * plan.Dm1:
        raise RuntimeError(f"mat1.size(-1) = {mat1.shape[-1]} does not match mat1Accum[-1] = {plan.Dm1}")
    if torch.is_grad_enabled() and (mat1.requires_grad or mat2.requires_grad):
        return _BlockGEMMFn.apply(mat1, mat2, plan, scale, bool(softmax))
    return plan.run(mat1, mat2, scale=scale)


def blockSoftmax(src: torch.Tensor, rowList: torch.Tensor, colList: torch.Tensor,
                 srcAccum: Optional[torch.Tensor] = None, *, scale: float = 1.0,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row softmax (last dim) of every packed block.

    ``src -> (H, sum rows_s*cols_s)``, result has the same shape; ``rowList =
    (rows_1, rows_2, ...)``, ``colList = (cols_1, ...)``; ``srcAccum = (0,
    rows_1*cols_1, ...)`` is optional.  ``out=src`` runs in place.
    """
    _check_operand("src", src)
    if rowList is None or colList is None:
        raise RuntimeError("blockSoftmax needs rowList and colList")
    key = ("smx", _key_of(rowList), _key_of(colList), _key_of(srcAccum), src.numel(), src.dtype, str(src.device))

    def build():
        rows, cols = _host_i64(rowList), _host_i64(colList)
        D = int(_host_i64(srcAccum)[-1]) if srcAccum is not None else int((rows * cols).sum())
        if D <= 0 or src.numel() % D:
            raise RuntimeError(f"src has {src.numel()} elements, not a multiple of the packed extent {D}")
        return SoftmaxPlan(rows, cols, src.numel() // D, src.dtype, accum=srcAccum, device=src.device)

    plan = _cached(key, build)
    if out is None and torch.is_grad_enabled() and src.requires_grad:
        return _BlockSoftmaxFn.apply(src, plan, scale)
    return plan.run(src, out=out, scale=scale)


def blockAttnScores(q: torch.Tensor, k: torch.Tensor, MList, NList, KList, scale: float = 1.0,
                    out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``softmax_rows(scale * Q_s K_s^T)`` for every segment in one pass: the
    fused form of ``blockSoftmax(blockGEMM(q, k, ...), MList, NList)``; the raw
    scores are never written to memory."""
    return blockGEMM(q, k, None, None, None, MList, NList, KList, False, False,
                     scale=scale, out_dtype=out_dtype, softmax=True)


class _BlockAttentionFn(torch.autograd.Function):
    """Fused forward.  The backward recomputes the probabilities with the fused scores operator and runs the softmax
    backward kernel and four blocked products (the same kernels the two-operator path differentiates with), so the
    probabilities exist in memory only during the backward pass.  Gradients have the layouts of q, k and v."""

    @staticmethod
    def forward(ctx, q, k, v, plan, scale):
        ctx.plan, ctx.scale = plan, scale
        ctx.save_for_backward(q, k, v)
        return plan.run(q, k, v, scale=scale)

    @staticmethod
    def backward(ctx, grad_out):
        q, k, v = ctx.saved_tensors
        plan, scale = ctx.plan, ctx.scale
        m, n = plan.M, plan.N
        dl = np.full_like(m, plan.d)
        with torch.no_grad():
            go = grad_out.contiguous().reshape(q.shape).to(q.dtype)
            p = blockGEMM(q, k, None, None, None, m, n, dl, False, False, scale=scale, softmax=True)   # (m, n)
            dv = blockGEMM(p, go, None, None, None, n, dl, m, True, True)           # P^T dO: (n, d)
            dp = blockGEMM(go, v, None, None, None, m, n, dl, False, False)         # dO V^T: (m, n)
            key = ("attn_bwd_smx", m.tobytes(), n.tobytes(), plan.H, q.dtype, str(q.device))
            sp = _cached(key, lambda: SoftmaxPlan(m, n, plan.H, q.dtype, device=q.device))
            ds = sp.run_backward(p, dp)                                              # d(scale * scores)
            dq = blockGEMM(ds, k, None, None, None, m, dl, n, False, True, scale=scale)   # dS K: (m, d)
            dk = blockGEMM(ds, q, None, None, None, n, dl, m, True, True, scale=scale)    # dS^T Q: (n, d)
        return dq.reshape(q.shape), dk.reshape(k.shape), dv.reshape(v.shape), None, None


def blockAttention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, MList, NList, scale: float = 1.0,
                   d: Optional[int] = None) -> torch.Tensor:
    """``softmax_rows(scale * Q_s K_s^T) V_s`` per segment: ``q -> (H, sum m_s*d)``, ``k, v -> (H, sum n_s*d)``, result
    ``(H, sum m_s*d)``, all packed head-major.  With 16-bit inputs and ``d`` 64 or 128 the batch runs as one kernel
    that never stores the probabilities (the pack kernel when every segment has at most 64 rows and columns and
    ``d = 64``, the tcgen05 attention kernel otherwise); any other batch is the composition
    ``blockGEMM(blockAttnScores(q, k), v, transpose2=True)`` of the two operators.  Carries autograd history: the
    backward pass recomputes the probabilities with the two-operator path."""
    for name, t in (("q", q), ("k", k), ("v", v)):
        _check_operand(name, t)
    M, N = _host_i64(MList), _host_i64(NList)
    rows_q, rows_kv = int(M.sum()), int(N.sum())
    if rows_q <= 0 or rows_kv <= 0:
        raise RuntimeError("blockAttention needs at least one query row and one key row")
    if d is None:
        # a (H, sum m_s * d) tensor tells d by its last extent; a flat one cannot (d and H only appear as a product)
        if q.dim() >= 2 and q.shape[-1] % rows_q == 0:
            d = int(q.shape[-1]) // rows_q
        else:
            raise RuntimeError("give the head dimension d (a flat tensor cannot tell it apart from the number of heads)")
    if q.numel() % (rows_q * d) or k.numel() != (q.numel() // (rows_q * d)) * rows_kv * d or v.numel() != k.numel():
        raise RuntimeError("q / k / v do not match the packed extents of the lists")
    H = q.numel() // (rows_q * d)
    fused = (d in (64, 128) and q.dtype in (torch.float16, torch.bfloat16) and k.dtype == q.dtype and v.dtype == q.dtype
             and int(N[M > 0].min() if (M > 0).any() else 1) >= 1)
    if fused:
        key = ("attn", M.tobytes(), N.tobytes(), H, d, q.dtype, str(q.device))
        try:
            plan = _cached(key, lambda: AttentionPlan(M, N, H, q.dtype, device=q.device, d=d))
            if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
                return _BlockAttentionFn.apply(q, k, v, plan, scale)
            return plan.run(q, k, v, scale=scale)
        except L.BlkError as e:
            if e.code != L.BLK_ERR_UNSUPPORTED:
                raise
    dl = np.full_like(M, d)
    p = blockGEMM(q, k, None, None, None, M, N, dl, False, False, scale=scale, softmax=True)
    return blockGEMM(p, v, None, None, None, M, dl, N, False, True)


def blockAttentionTokenMajor(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, nList, scale: float = 1.0) -> torch.Tensor:
    """Self-attention over a batch of graphs in the layout attention layers keep their activations in:
    ``q, k, v -> (sum n_s, H, d)`` (the nodes of all graphs in batch order), ``d`` 64 or 128, result of the same
    shape: ``out[rows of s] = softmax(scale * Q_s K_s^T) V_s`` per graph and head.  One kernel, no permuted copies,
    no probabilities in memory; graphs of any size, 16-bit inputs.  Forward only."""
    for name, t in (("q", q), ("k", k), ("v", v)):
        _check_operand(name, t)
    if q.dim() != 3 or q.shape != k.shape or q.shape != v.shape or q.shape[2] not in (64, 128):
        raise RuntimeError("q, k and v must all have shape (sum n, H, d), d 64 or 128")
    n = _host_i64(nList)
    H, d = int(q.shape[1]), int(q.shape[2])
    key = ("attn", n.tobytes(), n.tobytes(), H, d, q.dtype, str(q.device))
    plan = _cached(key, lambda: AttentionPlan(n, n, H, q.dtype, device=q.device, d=d))
    return plan.run_token_major(q, k, v, scale=scale)


def blockAttnScoresTokenMajor(q: torch.Tensor, k: torch.Tensor, nList, scale: float = 1.0,
                              out_dtype: Optional[torch.dtype] = None, softmax: bool = True) -> torch.Tensor:
    """``blockAttnScores`` for the layout attention inputs usually arrive in: ``q, k -> (sum n_s, H, d)``, the tokens
    of all segments in batch order.  The operands are read in place through strided tensor maps -- no permuted copy
    into head-major strips is made -- and the result is the packed head-major ``(H, sum n_s^2)`` buffer of
    ``blockAttnScores``.  Needs 16-bit inputs and ``d`` a multiple of 8 (16-byte rows for the tensor maps); with ``d = 32`` a batch
    with hundreds of segments of at most 64 tokens is refused (those run on a kernel that reads packed strips only).
    Forward only."""
    _check_operand("q", q)
    _check_operand("k", k)
    if q.dim() != 3 or q.shape != k.shape:
        raise RuntimeError("q and k must both have shape (sum n, H, d)")
    n = _host_i64(nList)
    H, d = int(q.shape[1]), int(q.shape[2])
    odt = out_dtype if out_dtype is not None else q.dtype
    key = ("tokmajor", n.tobytes(), H, d, q.dtype, odt, bool(softmax), str(q.device))
    plan = _cached(key, lambda: GemmPlan(n, n, np.full_like(n, d), H, q.dtype, odt, False, False, bool(softmax),
                                         device=q.device))
    return plan.run_token_major(q, k, scale=scale)


class _HostPipe:
    """Device-side staging of ``blockAttnScoresHost`` for one (lists, H, dtypes, device): a plan for a group of
    heads, two sets of device buffers and three streams (copy in, compute, copy out)."""

    def __init__(self, M, N, K, H, groups, dtype, odt, softmax, device):
        self.groups, self.Hg = groups, H // groups
        self.plan = GemmPlan(M, N, K, self.Hg, dtype, odt, False, False, softmax, device=device)
        p = self.plan
        self.bufs = [(torch.empty((self.Hg, p.Dm1), dtype=dtype, device=device),
                      torch.empty((self.Hg, p.Dm2), dtype=dtype, device=device),
                      torch.empty((self.Hg, p.Dout), dtype=odt, device=device)) for _ in range(2)]
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(device=device) for _ in range(3))


def blockAttnScoresHost(q: torch.Tensor, k: torch.Tensor, MList, NList, KList, scale: float = 1.0,
                        out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                        device=None, softmax: bool = True, head_groups: Optional[int] = None) -> torch.Tensor:
    """``blockAttnScores`` for operands and result that live in host memory.

    ``q -> (H, sum m_s*k_s)``, ``k -> (H, sum n_s*k_s)`` and the result ``(H, sum m_s*n_s)`` are host tensors
    (pinned memory makes the copies asynchronous).  The heads are processed in ``head_groups`` groups (default:
    one head per group, at most eight groups): while group g is computed, group g+1 is copied to the device and
    the result of group g-1 is copied back, so the transfer of the result and the arithmetic hide behind the
    transfer of the operands.  The call is ordered after work already queued on the current stream and the
    current stream waits for the last copy: synchronise it before reading ``out`` on the host.
    """
    for name, t in (("q", q), ("k", k)):
        if not isinstance(t, torch.Tensor) or t.is_cuda:
            raise RuntimeError(f"{name} must be a host tensor")
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous Tensor")
    if q.dtype != k.dtype:
        raise RuntimeError("q and k must have the same dtype")
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    odt = out_dtype if out_dtype is not None else q.dtype
    M, N, K = _host_i64(MList), _host_i64(NList), _host_i64(KList)
    Dm1, Dm2, Dout = int((M * K).sum()), int((N * K).sum()), int((M * N).sum())
    if Dm1 <= 0 or q.numel() % Dm1 or k.numel() != (q.numel() // Dm1) * Dm2:
        raise RuntimeError("q / k do not match the packed extents of the lists")
    H = q.numel() // Dm1
    groups = head_groups if head_groups is not None else next(g for g in range(min(H, 8), 0, -1) if H % g == 0)
    if groups < 1 or H % groups:
        raise RuntimeError(f"head_groups = {groups} does not divide H = {H}")
    if out is None:
        out = torch.empty((H, Dout), dtype=odt).pin_memory()
    elif out.is_cuda or not out.is_contiguous() or out.dtype != odt or out.numel() != H * Dout:
        raise RuntimeError("out must be a contiguous host tensor of the output dtype with H*Dout elements")
    key = ("hostpipe", M.tobytes(), N.tobytes(), K.tobytes(), H, groups, q.dtype, odt, bool(softmax), str(dev))
    pipe = _cached(key, lambda: _HostPipe(M, N, K, H, groups, q.dtype, odt, bool(softmax), dev))
    Hg = pipe.Hg
    qv, kv, ov = q.reshape(H, Dm1), k.reshape(H, Dm2), out.reshape(H, Dout)
    cur = torch.cuda.current_stream(dev)
    start = torch.cuda.Event()
    start.record(cur)
    for s in (pipe.s_in, pipe.s_run, pipe.s_out):
        s.wait_event(start)
    ran = [None, None]     # per buffer set: event after the kernels that read its operands
    drained = [None, None]  # per buffer set: event after the copy that read its result
    for g in range(groups):
        b = g & 1
        dq, dk, do = pipe.bufs[b]
        rows = slice(g * Hg, (g + 1) * Hg)
        with torch.cuda.stream(pipe.s_in):
            if ran[b] is not None:
                pipe.s_in.wait_event(ran[b])
            dq.copy_(qv[rows], non_blocking=True)
            dk.copy_(kv[rows], non_blocking=True)
            loaded = torch.cuda.Event()
            loaded.record(pipe.s_in)
        with torch.cuda.stream(pipe.s_run):
            pipe.s_run.wait_event(loaded)
            if drained[b] is not None:
                pipe.s_run.wait_event(drained[b])
            pipe.plan.run(dq, dk, out=do, scale=scale)
            ran[b] = torch.cuda.Event()
            ran[b].record(pipe.s_run)
        with torch.cuda.stream(pipe.s_out):
            pipe.s_out.wait_event(ran[b])
            ov[rows].copy_(do, non_blocking=True)
            drained[b] = torch.cuda.Event()
            drained[b].record(pipe.s_out)
    for ev in drained:
        if ev is not None:
            cur.wait_event(ev)
    return out
