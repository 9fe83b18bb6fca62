"""Batched symmetric eigensolver built from matrix products: spectral divide and conquer.

``torch.linalg.eigh`` (the reference's eigensolver, ``distributed_shampoo/preconditioner/
matrix_functions.py:725-770``) reduces to tridiagonal form with memory-bound Householder
updates, one matrix at a time.  On a tensor-core machine nearly all of the work of an
eigendecomposition can instead be matrix products over *all* factors of a refresh at once:

1. shift and scale:  ``X0 = (A - sigma I) / ||A - sigma I||_F`` with ``sigma = trace(A) / n``;
2. matrix sign function by a fixed schedule of odd quintic polynomials
   ``X <- X (a I + b X^2 + c X^4)`` (three symmetric products per iteration, no inverses);
   ``P = (I + sign(X0)) / 2`` is the orthogonal projector onto the eigenvalues above ``sigma``
   and ``k = ||P||_F^2`` its rank;
3. an orthonormal basis ``[V1 V2]`` adapted to the split: Householder QR of ``P Omega`` (``Omega``
   a fixed random ``n x k`` matrix), ``V1`` spans ``range(P)``, ``V2`` its complement;
4. the two half-size problems ``V1^T A V1`` and ``V2^T A V2`` go back on the work list; problems of
   size <= ``leaf`` are finished by the shared-memory Jacobi kernel.  The basis of every
   subproblem in the coordinates of its root matrix is carried along (``B <- B V``), so a leaf's
   eigenvectors are one more product.

A subproblem whose spread ``||A - sigma I||_F`` is at the rounding level of its root matrix is a
numerically multiple eigenvalue: any orthonormal basis serves and it is closed at once.  A sign
iteration that did not converge (an eigenvalue within ~1e-7 of the split point) is repeated with
a nudged split point.  Matrices the scheme gives up on are reported to the caller, which falls
back to the library eigensolver for them.

The driver below is written against a small backend interface.  ``TorchBackend`` implements it
with plain tensor operations on any device (the CPU tests run the whole algorithm through it);
``NativeBackend`` runs every product on the grouped tcgen05 GEMM, the QR panels on the
``householder_panel`` kernel and the leaves on ``jacobi_eigh``.
"""

from __future__ import annotations

import logging
import math
import os
import threading
from dataclasses import dataclass, field
from typing import Any

import torch
from torch import Tensor

logger: logging.Logger = logging.getLogger(__name__)

# Schedule of odd quintics p(x) = a x + b x^3 + c x^5 for the sign function of a matrix whose
# eigenvalues lie in [-1, 1]; every |x| >= 1e-7 ends within 1e-9 of 1.
#
# The first polynomial, applied 14 times, has the largest slope at 0 (3.19) among the quintics that
# are increasing on [0, 0.5], stay in [0.5, 1] on [0.5, 1] and have |p'| <= 2 there (a linear
# programme).  It is chosen for numerical stability, not for speed: a rounding error of the products
# that does not commute with the matrix is multiplied, per iteration, by the divided differences of
# p between pairs of eigenvalues.  Minimax ("equi-oscillating") polynomials reach 1 in 14 instead of
# 17 iterations but oscillate over the whole of [0, 1] with slopes up to 13 among eigenvalues that
# have already grown to O(1), which amplifies such errors by three orders of magnitude (measured:
# commutator ||[P, A]|| / ||A|| of 2e-4 instead of 3e-6 at the accuracy of the tf32x3 products).
# Here eigenvalues grow monotonically until they enter the band [0.5, 1], where slopes are bounded.
# The last three polynomials are minimax on [0.5, 1] and [0.95, 1] (small oscillation, slopes < 1)
# and the Newton-Schulz quintic.
_BAND = (3.19298245614035, -5.543859649122806, 3.087719298245614)
_FINISH = (
    (2.6073662581361705, -3.2052873333580942, 1.5974301564951396),
    (1.9203115684161138, -1.3422577427092492, 0.42194449535688716),
    (1.875, -1.25, 0.375),
)
SIGN_SCHEDULE: tuple[tuple[float, float, float], ...] = (_BAND,) * 14 + _FINISH
# The 14 band iterations are what an eigenvalue 1e-7 away from the split point needs; the closest
# eigenvalue of a real subproblem is typically 1e-5 to 1e-3 away (5 to 9 iterations).  So the
# iteration runs in two stages: 9 band iterations and the finishing three, then, only for the
# subproblems whose projector is not idempotent yet (an eigenvalue still between 0 and 1 shows in
# trace(P) - ||P||_F^2), 5 more band iterations and the finishing three from X = 2 P - I.
# OB200_SIGN_STAGE1 overrides the length of the first stage (14 gives the single fixed schedule).
_STAGE1 = min(max(int(os.environ.get("OB200_SIGN_STAGE1", "9")), 1), 14)
SIGN_STAGES: tuple[tuple[tuple[float, float, float], ...], ...] = ((_BAND,) * _STAGE1 + _FINISH,) + (
    ((_BAND,) * (14 - _STAGE1) + _FINISH,) if _STAGE1 < 14 else ()
)

LEAF = 128  # largest problem the Jacobi kernel takes
_MAX_ATTEMPTS = 3  # sign computations per subproblem before its root is given up
_MAX_ROUNDS = 40  # rounds of the work list before the remaining roots are given up
_IDEMPOTENCY_TOL = 0.05  # bound on |trace(P) - ||P||_F^2| = |sum p (1 - p)| over the eigenvalues p of P
_NUDGE = 3e-5  # relative shift of the split point for a repeated sign computation


@dataclass
class Sub:
    """One symmetric subproblem: ``A`` (n x n) is the restriction of root matrix ``root`` to the
    subspace spanned by the columns of ``B`` (d_root x n); its eigenvalues belong at positions
    ``offset .. offset + n`` of the root's (unsorted) spectrum."""

    root: int
    n: int
    offset: int
    A: Any = None  # backend handle of the matrix
    B: Any = None  # backend handle of the basis; None for a root (identity)
    attempt: int = 0  # sign computations of this subproblem that did not yield a projector
    mean: float = 0.0  # trace / n
    mean_spread: float = 0.0  # ||A - mean I||_F
    sigma: float = 0.0  # split point
    spread: float = 0.0  # ||A - sigma I||_F
    lo: float = -math.inf  # known bounds of the eigenvalues (from the splits that produced the subproblem)
    hi: float = math.inf
    span: tuple[int, int] | None = None  # positions of its eigenvalues in the root's hint, descending order
    rule: str = "mean"  # how sigma was chosen: "mean", "hint", "geometric"
    one_sided: bool = False  # a hinted or geometric split point failed here: the mean from now on
    rank: int = 0
    idem_err: float = 0.0
    extra: dict = field(default_factory=dict)  # backend scratch


class TorchBackend:
    """Reference implementation of the backend interface with plain tensor operations."""

    def __init__(self, device: torch.device, dtype: torch.dtype = torch.float32, seed: int = 1234) -> None:
        self.device, self.dtype = device, dtype
        self._omega: Tensor | None = None
        self._seed = seed
        self.passes = 2
        self.sign_stages_run = [0] * len(SIGN_STAGES)  # subproblems that went through each stage

    # -- set-up -----------------------------------------------------------------------------
    def begin(self, mats: list[Tensor]) -> list[Sub]:
        dmax = max(m.shape[0] for m in mats)
        gen = torch.Generator(device="cpu").manual_seed(self._seed)
        self._omega = torch.randn(dmax, dmax, generator=gen).to(device=self.device, dtype=self.dtype)
        self.lams = [torch.zeros(m.shape[0], device=self.device, dtype=self.dtype) for m in mats]
        self.vecs = [torch.zeros(m.shape[0], m.shape[0], device=self.device, dtype=self.dtype) for m in mats]
        self.root_norms = [float(torch.linalg.norm(m)) for m in mats]
        return [Sub(root=i, n=m.shape[0], offset=0, A=m.to(self.dtype).clone()) for i, m in enumerate(mats)]

    # -- one round ----------------------------------------------------------------------------
    def measure(self, subs: list[Sub]) -> None:
        """mean = trace / n and spread = ||A - mean I||_F (the driver derives the split point)."""
        for s in subs:
            mean = float(torch.trace(s.A)) / s.n
            shifted = s.A - mean * torch.eye(s.n, device=self.device, dtype=self.dtype)
            s.mean, s.mean_spread = mean, float(torch.linalg.norm(shifted))

    def sign_projector(self, subs: list[Sub]) -> None:
        """P = (I + sign(A - sigma I)) / 2, rank = ||P||_F^2, idem_err = trace(P) - ||P||_F^2."""
        for s in subs:
            eye = torch.eye(s.n, device=self.device, dtype=self.dtype)
            X = (s.A - s.sigma * eye) / s.spread
            for stage, schedule in enumerate(SIGN_STAGES):
                for a, b, c in schedule:
                    Y = X @ X
                    Y = 0.5 * (Y + Y.T)
                    W = c * (Y @ Y) + b * Y + a * eye
                    W = 0.5 * (W + W.T)
                    X = X @ W
                    X = 0.5 * (X + X.T)
                P = 0.5 * X + 0.5 * eye
                fro2 = float((P * P).sum())
                s.rank = int(round(fro2))
                s.idem_err = float(torch.trace(P)) - fro2
                self.sign_stages_run[stage] += 1
                if abs(s.idem_err) <= _IDEMPOTENCY_TOL:
                    break
            s.extra["P"] = P

    def split_basis(self, subs: list[Sub]) -> None:
        """Qt (n x n, rows orthonormal): the first ``rank`` rows span range(P)."""
        for s in subs:
            k, n = s.rank, s.n
            P = s.extra.pop("P")
            Y = P @ self._omega[:n, :k]  # n x k
            Q, _ = torch.linalg.qr(Y, mode="complete")
            for _ in range(self.passes - 1):
                Q, _ = torch.linalg.qr(P @ Q[:, :k], mode="complete")
            s.extra["Qt"] = Q.T.contiguous()

    def project(self, subs: list[Sub]) -> list[Sub]:
        """Children (V1^T A V1, above sigma) and (V2^T A V2, below) with their bases B V."""
        children = []
        for s in subs:
            Qt = s.extra.pop("Qt")
            k = s.rank
            for rows, off in ((slice(0, k), s.offset), (slice(k, s.n), s.offset + k)):
                Vt = Qt[rows]
                A_child = Vt @ s.A @ Vt.T
                A_child = 0.5 * (A_child + A_child.T)
                B_child = Vt.T.contiguous() if s.B is None else s.B @ Vt.T
                children.append(Sub(root=s.root, n=Vt.shape[0], offset=off, A=A_child, B=B_child))
            s.A = s.B = None
        return children

    def close_scalar(self, subs: list[Sub]) -> None:
        """Numerically multiple eigenvalue: eigenvalues = diag(A), eigenvectors = columns of B."""
        for s in subs:
            self.lams[s.root][s.offset : s.offset + s.n] = torch.diagonal(s.A)
            self.vecs[s.root][:, s.offset : s.offset + s.n] = (
                torch.eye(s.n, device=self.device, dtype=self.dtype) if s.B is None else s.B
            )

    def close_leaves(self, subs: list[Sub]) -> list[int]:
        """Eigendecomposition of the small problems; returns the roots of those that failed."""
        for s in subs:
            lam, Q = torch.linalg.eigh(s.A)
            self.lams[s.root][s.offset : s.offset + s.n] = lam
            self.vecs[s.root][:, s.offset : s.offset + s.n] = Q if s.B is None else s.B @ Q
        return []

    def finish(self, roots_ok: list[bool]) -> tuple[list[Tensor | None], list[Tensor | None]]:
        lams: list[Tensor | None] = []
        vecs: list[Tensor | None] = []
        for ok, lam, Q in zip(roots_ok, self.lams, self.vecs, strict=True):
            if not ok:
                lams.append(None)
                vecs.append(None)
                continue
            order = torch.argsort(lam, stable=True)
            lams.append(lam[order])
            vecs.append(Q[:, order].contiguous())
        return lams, vecs


_HEAVY_TAIL = 8.0  # n * sum(lambda^2) / sum(lambda)^2 above which the mean says little about the median
_SAFE_GAP = 4e-6  # smallest gap, relative to the spread, in which a hinted split point is placed
_WIDE_RANGE = 1e3  # hi / lo above which a heavy-tailed spectrum is split at the geometric mean of its bounds


def plan_split(s: Sub, hint: Any, floor: float) -> None:
    """Choose the split point ``s.sigma`` (and ``s.spread = ||A - sigma I||_F``) of a measured
    subproblem.  The mean of the eigenvalues always has eigenvalues on both sides, but on the
    heavy-tailed spectra of Kronecker factors (a handful of dominant eigenvalues, many decades of
    tail, often a numerically null cluster) it isolates a few eigenvalues per round.  In order:

    - after a split point that left everything on one side, or without better knowledge: the mean;
    - with a hint (eigenvalue estimates of the same matrix from an earlier decomposition, any
      positive scale, sorted descending): the largest gap in the middle third of the subproblem's
      part of the hint, rescaled by the current trace: balanced splits and the null cluster comes
      off in one piece;
    - heavy tail and bounds (from the splits above, the norm, and the rounding floor) that span more
      than three decades: the geometric mean of the bounds;
    - a sign iteration that did not converge is repeated with the point nudged by 3e-5 of the spread.
    """
    n, mean, spread = s.n, s.mean, s.mean_spread
    sigma, rule = mean, "mean"
    hi = min(s.hi, mean + spread)
    lo = max(s.lo, mean - spread)
    if not s.one_sided:
        span = s.span
        if hint is not None and span is not None and span[1] - span[0] == n and n >= 4:
            part = hint[span[0] : span[1]]
            total = float(part.sum())
            if total > 0.0 and mean > 0.0:
                scale = mean * n / total
                # Splitting between positions m - 1 and m (m eigenvalues above) is only safe where the
                # gap is resolved by the sign iteration: eigenvalues closer to the split point than
                # ~1e-7 of the spread do not converge.  Among the safe positions take the one that
                # balances the two halves best (cost m^3 + (n - m)^3).
                gaps = (part[:-1] - part[1:]) * scale  # gaps[m - 1]: between positions m - 1 and m
                safe = torch.nonzero(gaps >= _SAFE_GAP * spread).flatten() + 1
                if safe.numel():
                    m = int(safe[(safe - n / 2).abs().argmin()])
                    if min(m, n - m) >= max(2, n // 16):  # a split that moves less is left to the other rules
                        cand = 0.5 * float(part[m - 1] + part[m]) * scale
                        if lo < cand < hi:
                            sigma, rule = cand, "hint"
        if rule == "mean" and mean > 0.0:
            ratio = (spread * spread + n * mean * mean) / (n * mean * mean)
            low = max(lo, floor)
            if ratio > _HEAVY_TAIL and hi > 0.0 and hi / low > _WIDE_RANGE:
                cand = math.sqrt(hi * low)
                if cand < mean:
                    sigma, rule = cand, "geometric"
    if s.attempt:
        sigma += _NUDGE * s.attempt * max(spread, abs(sigma - mean)) * (1 if s.attempt % 2 else -1)
    shift = sigma - mean
    s.sigma, s.rule = sigma, rule
    s.spread = math.sqrt(spread * spread + n * shift * shift)  # trace(A - mean I) = 0


class _Timed:
    """Wraps a backend whose ``profile`` attribute is a dict: every phase is bracketed by a device
    synchronisation and its wall time is added to ``profile[phase]`` (diagnostics only; the
    synchronisations serialise host and device)."""

    def __init__(self, backend: Any) -> None:
        self._backend = backend

    def __getattr__(self, name: str) -> Any:
        attr = getattr(self._backend, name)
        if not callable(attr) or name.startswith("_"):
            return attr
        import time

        def timed(*args: Any, **kwargs: Any) -> Any:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            t0 = time.perf_counter()
            out = attr(*args, **kwargs)
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            prof = self._backend.profile
            ms = (time.perf_counter() - t0) * 1e3
            prof[name] = prof.get(name, 0.0) + ms
            if args and isinstance(args[0], list) and args[0] and isinstance(args[0][0], Sub):
                # per call: number of subproblems, their mean size, milliseconds, sum n^3 and sum n^2 rank (in 1e9)
                subs = args[0]
                prof.setdefault("calls", []).append((
                    name, len(subs), round(sum(s.n for s in subs) / len(subs)), round(ms, 2),
                    round(sum(float(s.n) ** 3 for s in subs) / 1e9, 2),
                    round(sum(float(s.n) ** 2 * max(s.rank, 0) for s in subs) / 1e9, 2),
                ))
            return out

        return timed


def eigh_divide_and_conquer(
    backend: Any, mats: list[Tensor], leaf: int = LEAF, scalar_tol: float = 4.0, hints: list[Any] | None = None
) -> tuple[list[Tensor | None], list[Tensor | None], dict[str, Any]]:
    """Eigendecompositions (ascending eigenvalues, eigenvectors as columns) of the symmetric
    matrices ``mats``, all advanced together.  Returns ``(eigenvalues, eigenvectors, info)``; the
    entries of matrices the scheme gave up on are ``None`` and their indices are in
    ``info["failed"]``.

    ``scalar_tol``: a subproblem is closed as a multiple eigenvalue when its spread is below
    ``scalar_tol * eps * ||root matrix||_F``.

    ``hints``: per matrix ``None`` or a 1-D CPU tensor of eigenvalue estimates of the same size (any
    positive scale, any order), e.g. the eigenvalues found at the previous refresh; they only steer
    the choice of split points (``plan_split``)."""
    eps = torch.finfo(torch.float32).eps
    backend = _Timed(backend) if getattr(backend, "profile", None) is not None else backend
    work = backend.begin(mats)
    plans: list[Any] = [None] * len(mats)
    if hints is not None:
        for i, h in enumerate(hints):
            if h is not None and h.numel() == mats[i].shape[0]:
                plans[i] = torch.sort(h.detach().to(device="cpu", dtype=torch.float64), descending=True).values
    for s in work:
        if plans[s.root] is not None:
            s.span = (0, s.n)
    one_sided = 0
    failed: set[int] = set()
    reasons: dict[int, str] = {}
    rounds = 0
    signs = 0
    cubes = 0.0  # sum of n^3 over all sign computations: the unit the cost of a refresh scales with
    while work:
        rounds += 1
        work = [s for s in work if s.root not in failed]
        leaves = [s for s in work if s.n <= leaf]
        big = [s for s in work if s.n > leaf]
        if leaves:
            failed.update(backend.close_leaves(leaves))
        if not big:
            break
        if rounds > _MAX_ROUNDS:
            for s in big:
                failed.add(s.root)
                reasons.setdefault(s.root, f"still splitting after {_MAX_ROUNDS} rounds (subproblem of size {s.n})")
            break
        backend.measure(big)
        is_scalar = lambda s: s.mean_spread <= scalar_tol * eps * backend.root_norms[s.root] or s.mean_spread == 0.0  # noqa: E731
        scalar = [s for s in big if is_scalar(s)]
        if scalar:
            backend.close_scalar(scalar)
        active = [s for s in big if not is_scalar(s)]
        for s in active:
            plan_split(s, plans[s.root], scalar_tol * eps * backend.root_norms[s.root])
        if not active:
            work = []
            continue
        backend.sign_projector(active)
        signs += len(active)
        cubes += sum(float(s.n) ** 3 for s in active)
        good, retry = [], []
        for s in active:
            converged = abs(s.idem_err) <= _IDEMPOTENCY_TOL  # False for NaN
            if converged and 0 < s.rank < s.n:
                good.append(s)
                continue
            if s.rule != "mean":
                # A hinted or geometric split point that left every eigenvalue on one side (a bound
                # learned) or landed where eigenvalues crowd (no projector): a sign computation
                # spent; the subproblem continues with the mean, which cannot fail the first way.
                if converged and s.rank <= 0:
                    s.hi = min(s.hi, s.sigma)
                elif converged:
                    s.lo = max(s.lo, s.sigma)
                s.one_sided = True
                s.extra.clear()
                retry.append(s)
                one_sided += 1
                continue
            s.attempt += 1
            s.extra.clear()
            if s.attempt >= _MAX_ATTEMPTS:
                failed.add(s.root)
                reasons.setdefault(
                    s.root,
                    f"no projector after {_MAX_ATTEMPTS} sign computations: subproblem n={s.n} rank={s.rank} "
                    f"idempotency defect={s.idem_err:.3g} spread={s.spread:.3g} (root norm {backend.root_norms[s.root]:.3g})",
                )
            else:
                retry.append(s)
        children: list[Sub] = []
        if good:
            backend.split_basis(good)
            split_of = {(s.root, s.offset): s for s in good}
            children = backend.project(good)
            for c in children:
                parent = split_of.get((c.root, c.offset))
                above = parent is not None  # the child of the eigenvalues above sigma keeps the parent's offset
                if parent is None:
                    parent = next(p for p in good if p.root == c.root and p.offset + p.rank == c.offset)
                c.lo, c.hi = (parent.sigma, parent.hi) if above else (parent.lo, parent.sigma)
                if parent.span is not None:
                    a = parent.span[0]
                    c.span = (a, a + parent.rank) if above else (a + parent.rank, parent.span[1])
        work = retry + children
    ok = [i not in failed for i in range(len(mats))]
    lams, vecs = backend.finish(ok)
    return lams, vecs, {
        "failed": sorted(failed), "rounds": rounds, "sign_computations": signs, "sign_cubes": cubes, "reasons": reasons,
        "one_sided_splits": one_sided,  # hinted / geometric points that had to be abandoned
        "sign_stages": list(getattr(backend, "sign_stages_run", [])),  # subproblems through each stage of the schedule
    }


# ----------------------------------------------------------------------------------------------
# The sm_100a backend
# ----------------------------------------------------------------------------------------------
def _pad4(n: int) -> int:
    return (n + 3) // 4 * 4


class _Mat:
    """A matrix in padded storage, as the plain array and/or as the tf32 (hi, lo) operand pair.
    ``rows x cols`` with row pitch ``pad4(cols)``; the attributes are the exact-size views."""

    __slots__ = ("rows", "cols", "plain", "hi", "lo")

    def __init__(self, rows: int, cols: int, device: torch.device, plain: bool = True, pair: bool = True) -> None:
        self.rows, self.cols = rows, cols
        ld = _pad4(cols)
        count = int(plain) + 2 * int(pair)
        # one allocation for the arrays of this matrix; each array starts on a 16-byte boundary
        block = torch.empty(count * rows * ld, device=device, dtype=torch.float32)
        views = [torch.as_strided(block, (rows, cols), (ld, 1), k * rows * ld) for k in range(count)]
        self.plain = views.pop(0) if plain else None
        self.hi, self.lo = (views[0], views[1]) if pair else (None, None)


def _mats(ext: Any, device: torch.device, shapes: list[tuple[int, int]], plain: bool = True, pair: bool = True) -> list[_Mat]:
    """``_Mat(rows, cols, device, plain, pair)`` for every shape out of one allocation, the views
    made by the extension: a refresh creates tens of thousands of scratch matrices, and one
    allocation plus three views each in Python was a third of its host time.  The matrices of a
    batch share their storage, so a batch should hold arrays of one lifetime."""
    make = getattr(ext, "alloc_mat_batch", None)
    if make is None or not shapes:
        return [_Mat(r, c, device, plain=plain, pair=pair) for r, c in shapes]
    out = []
    new = _Mat.__new__
    for (r, c), (p, hi, lo) in zip(shapes, make([r for r, _ in shapes], [c for _, c in shapes], plain, pair, device)):
        m = new(_Mat)
        m.rows, m.cols, m.plain, m.hi, m.lo = r, c, p, hi, lo
        out.append(m)
    return out


_OMEGA_CACHE: dict[tuple, _Mat] = {}
_OMEGA_LOCK = threading.Lock()


def prepare_test_matrix(ext: Any, device: torch.device, dmax: int, seed: int = 1234) -> _Mat:
    """The random test matrix Omega^T (rows are the columns of Omega) as an operand pair, at least
    ``dmax`` square; one per device and seed is kept, and a larger one serves smaller requests (the
    solver only uses leading blocks).  Callers that run several solvers concurrently call this
    first with the largest size so that the solvers find it made."""
    key = (device.type, device.index, seed)
    with _OMEGA_LOCK:
        om = _OMEGA_CACHE.get(key)
        if om is None or om.rows < dmax:
            gen = torch.Generator(device="cpu").manual_seed(seed)
            omega_t = torch.randn(dmax, dmax, generator=gen).to(device)
            om = _Mat(dmax, dmax, device, plain=False)
            ext.tf32_split(omega_t, om.hi, om.lo)
            _OMEGA_CACHE[key] = om
        return om



class NativeBackend:
    """Backend of ``eigh_divide_and_conquer`` on the sm_100a kernels.  Every product is a problem of
    a grouped tcgen05 launch over all subproblems of a round (symmetric results compute only the
    tiles on or above the diagonal); the host reads the device twice per round (split points and
    spreads; ranks and idempotency defects) and once at the end (leaf convergence)."""

    def __init__(self, ext: Any, device: torch.device, status: Tensor | None = None, range_passes: int = 2, seed: int = 1234,
                 polish: str = "householder") -> None:
        assert polish in ("householder", "newton_schulz")
        self.polish = polish  # how the second range pass is made (see _polish)
        self.ext, self.device = ext, device
        self.status = status if status is not None else torch.zeros(1, dtype=torch.int32, device=device)
        self.range_passes = range_passes
        self._seed = seed
        self._leaf_sweeps: list[tuple[list[Sub], Tensor]] = []
        self.profile: dict[str, float] | None = None  # set to {} to collect per-phase times
        self.jacobi_max_sweeps = 24
        self.jacobi_tolerance = 2e-6
        self.jacobi_shift = 1.5  # second attempt of a leaf the Jacobi kernel did not settle on (see finish)
        self.leaves_retried = 0
        self.sign_stages_run = [0] * len(SIGN_STAGES)  # subproblems that went through each stage

    # -- helpers ----------------------------------------------------------------------------
    def _gemm(self, specs: list[tuple], alpha: float = 1.0, beta: float = 0.0, gamma: float = 0.0) -> None:
        if specs:
            plan = self.ext.build_gemm_plan(specs)
            self.ext.run_gemm_plan(*plan, alpha, beta, True, self.status, gamma)

    def _spec(self, a: _Mat, b: _Mat, out: _Mat | None, c: Tensor | None = None, flags: int = 0, sumsq: Tensor | None = None,
              sym: bool = False, c_ld: int = 0) -> tuple:
        """C = alpha A B^T (+ beta C) with the (hi, lo) pair of the result written to ``out``."""
        F = self.ext
        if sym:
            flags |= F.FLAG_MIRROR
        d_hi = d_lo = None
        ldd = 0
        if out is not None and out.hi is not None:
            flags |= F.FLAG_SPLIT_OUT
            d_hi, d_lo, ldd = out.hi, out.lo, out.hi.stride(0)
        if c is None:
            flags |= F.FLAG_NO_C
        else:
            c_ld = c.stride(0)
        return (a.hi, a.lo, b.hi, b.lo, c, d_hi, d_lo, sumsq, c_ld, ldd, flags, sym)

    # -- set-up -----------------------------------------------------------------------------
    def begin(self, mats: list[Tensor]) -> list[Sub]:
        ext, dev = self.ext, self.device
        dmax = max(m.shape[0] for m in mats)
        self._omega_t = prepare_test_matrix(ext, dev, dmax, self._seed)
        self.lams = [torch.zeros(m.shape[0], device=dev) for m in mats]
        self.vecs = [torch.zeros(m.shape[0], m.shape[0], device=dev) for m in mats]
        self.root_norms = torch.stack(torch._foreach_norm(list(mats))).cpu().tolist()
        subs = []
        for i, (m, A) in enumerate(zip(mats, _mats(ext, dev, [(m.shape[0], m.shape[0]) for m in mats]), strict=True)):
            n = m.shape[0]
            A.plain.copy_(m)
            ext.tf32_split(A.plain, A.hi, A.lo)
            subs.append(Sub(root=i, n=n, offset=0, A=A))
        self._leaf_sweeps = []
        return subs

    # -- one round ----------------------------------------------------------------------------
    def measure(self, subs: list[Sub]) -> None:
        ext = self.ext
        stats = torch.zeros(len(subs), 2, device=self.device)
        table = ext.build_sym_table([(s.A.plain, None, None, stats[i], 0.0, 0.0) for i, s in enumerate(subs)])
        ext.sym_measure(table[0], len(subs))
        for s, (mean, spread) in zip(subs, stats.cpu().tolist(), strict=True):
            s.mean, s.mean_spread = mean, spread

    def sign_projector(self, subs: list[Sub]) -> None:
        ext, dev = self.ext, self.device
        start = _mats(ext, dev, [(s.n, s.n) for s in subs], plain=False)
        table = ext.build_sym_table(
            [(s.A.plain, start[i].hi, start[i].lo, None, 1.0 / s.spread, -s.sigma / s.spread) for i, s in enumerate(subs)]
        )
        ext.shift_scale_split(*table)
        todo, X0 = list(subs), start
        for stage, schedule in enumerate(SIGN_STAGES):
            projectors = self._sign_stage(todo, X0, schedule)
            self.sign_stages_run[stage] += len(todo)
            again, again_x = [], []
            for s, P in zip(todo, projectors, strict=True):
                s.extra["P"] = P
                if stage + 1 < len(SIGN_STAGES) and s.rank >= 0 and not abs(s.idem_err) <= _IDEMPOTENCY_TOL:
                    # not a projector yet: X = 2 P - I goes through the next stage (an elementwise pass)
                    X = _Mat(s.n, s.n, dev)
                    torch.add(P.hi, P.lo, out=X.plain)
                    again.append(s)
                    again_x.append(X)
            if not again:
                break
            table = ext.build_sym_table([(X.plain, X.hi, X.lo, None, 2.0, -1.0) for X in again_x])
            ext.shift_scale_split(*table)
            todo, X0 = again, again_x

    def _sign_stage(self, subs: list[Sub], X0: list[_Mat], schedule: tuple) -> list[_Mat]:
        """The polynomials of ``schedule`` applied to the iterates ``X0`` (operand pairs), the last
        one fused with P = X / 2 + I / 2; sets ``rank`` and ``idem_err`` of ``subs`` from the
        epilogue's ||P||_F^2 and trace(P) and returns the projectors."""
        ext, dev, F = self.ext, self.device, self.ext
        square = [(s.n, s.n) for s in subs]
        X = [X0, _mats(ext, dev, square, plain=False)]
        Y = _mats(ext, dev, square)
        W = _mats(ext, dev, square, plain=False)
        stats = torch.zeros(len(subs), 2, device=dev)
        idx = range(len(subs))
        plans = []
        for cur in (0, 1):
            nxt = cur ^ 1
            g1 = [self._spec(X[cur][i], X[cur][i], Y[i], c=Y[i].plain, sym=True) for i in idx]
            # W = c Y Y + b Y + a I: beta applies to the plain copy of Y that C holds
            g2 = [self._spec(Y[i], Y[i], W[i], c=Y[i].plain, flags=F.FLAG_ADD_DIAG, sym=True) for i in idx]
            g3 = [self._spec(X[cur][i], W[i], X[nxt][i], sym=True) for i in idx]
            plans.append([ext.build_gemm_plan(g) for g in (g1, g2, g3)])
        cur = 0
        last = len(schedule) - 1
        for it, (a, b, c) in enumerate(schedule):
            p1, p2, p3 = plans[cur]
            ext.run_gemm_plan(*p1, 1.0, 0.0, True, self.status)
            ext.run_gemm_plan(*p2, c, b, True, self.status, a)
            if it == last:
                # P = X W / 2 + I / 2 with ||P||_F^2 and trace(P) from the epilogue
                final = [
                    self._spec(X[cur][i], W[i], X[cur ^ 1][i], flags=F.FLAG_ADD_DIAG | F.FLAG_SUMSQ | F.FLAG_TRACE,
                               sumsq=stats[i], sym=True)
                    for i in idx
                ]
                self._gemm(final, 0.5, 0.0, 0.5)
            else:
                ext.run_gemm_plan(*p3, 1.0, 0.0, True, self.status)
            cur ^= 1
        for s, (fro2, trace) in zip(subs, stats.cpu().tolist(), strict=True):
            finite = fro2 == fro2 and abs(fro2) != float("inf")
            s.rank = int(round(fro2)) if finite else -1
            s.idem_err = trace - fro2 if finite else float("nan")
        return [X[cur][i] for i in idx]

    def split_basis(self, subs: list[Sub]) -> None:
        ext, dev = self.ext, self.device
        om = self._omega_t
        qr_specs, g = [], []
        # A Householder second pass only reads V1, the first rank rows of this pass's Q^T: the
        # accumulation then produces those rows only.
        head_only = self.range_passes > 1 and self.polish == "householder"
        Yts = _mats(ext, dev, [(s.rank, s.n) for s in subs], pair=False)  # rows: the columns of P Omega
        Zts = _mats(ext, dev, [(s.rank if head_only else s.n, s.n) for s in subs])
        for s, Yt, Zt in zip(subs, Yts, Zts, strict=True):
            k, n = s.rank, s.n
            P = s.extra.pop("P")
            s.extra["Qt"] = Zt
            g.append((om.hi, om.lo, P.hi, P.lo, Yt.plain, None, None, None, Yt.plain.stride(0), 0,
                      0, False, None, (0, 0, 0, 0, k, n, n)))
            qr_specs.append((Yt.plain, n, k, Zt.plain, Zt.hi, Zt.lo, k if head_only else n))
            s.extra["P_keep"] = P
        # the Omega view ends before its array along K unless n == dmax: K = n must then be a multiple of 32;
        # otherwise fall back to a sliced operand (its own tensor map)
        fixed = []
        for spec, s in zip(g, subs, strict=True):
            n, k = s.n, s.rank
            if n == om.cols or n % 32 == 0:
                fixed.append(spec)
            else:
                fixed.append((om.hi[:k, :n], om.lo[:k, :n]) + spec[2:13] + (None,))
        self._gemm(fixed)
        ext.householder_qr(qr_specs)
        if self.range_passes > 1 and self.polish == "newton_schulz":
            self._polish(subs)
        for _ in range(self.range_passes - 1 if self.polish == "householder" else 0):
            # One more pass from the orthonormal basis just found: Y <- P V1, whose conditioning is 1.
            g, qr_specs = [], []
            Yts = _mats(ext, dev, [(s.rank, s.n) for s in subs], pair=False)
            Zts = _mats(ext, dev, [(s.n, s.n) for s in subs])
            for s, Yt, Zt in zip(subs, Yts, Zts, strict=True):
                k, n = s.rank, s.n
                P, Zt_old = s.extra["P_keep"], s.extra["Qt"]
                v1 = _Mat.__new__(_Mat)
                v1.rows, v1.cols, v1.plain, v1.hi, v1.lo = k, n, None, Zt_old.hi[:k], Zt_old.lo[:k]
                g.append(self._spec(v1, P, None, c=Yt.plain))
                qr_specs.append((Yt.plain, n, k, Zt.plain, Zt.hi, Zt.lo))
                s.extra["Qt"] = Zt
            self._gemm(g)
            ext.householder_qr(qr_specs)
        for s in subs:
            s.extra.pop("P_keep")

    def _polish(self, subs: list[Sub]) -> None:
        """Second range pass as matrix products.  With Q = [V1 V2] from the Householder pass,
        Z = [P V1, (I - P) V2] re-projects both halves onto the invariant subspaces (its columns are
        orthonormal up to the rounding of the first pass times the conditioning of P Omega), and one
        Newton-Schulz step Z (3 I - Z^T Z) / 2 squares that defect.  2.5 n^3 on the tensor cores
        instead of a second Householder factorisation.  All arrays hold the transposes (rows = basis
        vectors)."""
        ext, dev, F = self.ext, self.device, self.ext
        head, tail, gram, last, tr = [], [], [], [], []
        for s in subs:
            k, n = s.rank, s.n
            P, old = s.extra["P_keep"], s.extra["Qt"]
            Z, S, ZT, new = (_Mat(n, n, dev, plain=False) for _ in range(4))

            def rows(m: _Mat, r0: int, r1: int, with_plain: bool = False) -> _Mat:
                v = _Mat.__new__(_Mat)
                v.rows, v.cols, v.hi, v.lo = r1 - r0, m.cols, m.hi[r0:r1], m.lo[r0:r1]
                v.plain = m.plain[r0:r1] if with_plain else None
                return v

            if k > 0:
                head.append(self._spec(rows(old, 0, k), P, rows(Z, 0, k)))
            if k < n:  # (I - P) V2 = V2 - P V2: beta = 1 on the plain copy of the old rows
                tail.append(self._spec(rows(old, k, n), P, rows(Z, k, n), c=old.plain[k:n]))
            gram.append(self._spec(Z, Z, S, flags=F.FLAG_ADD_DIAG, sym=True))
            tr += [(Z.hi, ZT.hi, None, None), (Z.lo, ZT.lo, None, None)]
            last.append(self._spec(S, ZT, new))
            s.extra["Qt"] = new
        self._gemm(head)
        self._gemm(tail, -1.0, 1.0)
        self._gemm(gram, -0.5, 0.0, 1.5)
        ext.transpose_split(*ext.build_transpose_table(tr))
        self._gemm(last)

    def project(self, subs: list[Sub]) -> list[Sub]:
        ext, dev = self.ext, self.device
        children: list[Sub] = []
        g1, g2, g3 = [], [], []
        halves = [(m, s.n, self.lams[s.root].shape[0]) for s in subs for m in (s.rank, s.n - s.rank)]
        Ts = iter(_mats(ext, dev, [(m, n) for m, n, _ in halves], plain=False))
        Acs = iter(_mats(ext, dev, [(m, m) for m, _, _ in halves]))
        Bcs = iter(_mats(ext, dev, [(d, m) for m, _, d in halves]))
        for s in subs:
            Qt = s.extra.pop("Qt")
            k, n = s.rank, s.n
            for r0, r1, off in ((0, k, s.offset), (k, n, s.offset + k)):
                m = r1 - r0
                vt = _Mat.__new__(_Mat)
                vt.rows, vt.cols, vt.plain, vt.hi, vt.lo = m, n, None, Qt.hi[r0:r1], Qt.lo[r0:r1]
                T, Ac, Bc = next(Ts), next(Acs), next(Bcs)  # V^T A, the child, its basis
                g1.append(self._spec(vt, s.A, T))
                g2.append(self._spec(T, vt, Ac, c=Ac.plain, sym=True))
                if s.B is None:
                    # B = I V: a transposed copy of V^T
                    s.extra.setdefault("transposes", []).append((vt, Bc))
                else:
                    g3.append(self._spec(s.B, vt, Bc, c=Bc.plain))
                children.append(Sub(root=s.root, n=m, offset=off, A=Ac, B=Bc))
        self._gemm(g1)
        self._gemm(g2)
        self._gemm(g3)
        tr = [(vt.hi, vt.lo, Bc) for s in subs for vt, Bc in s.extra.pop("transposes", [])]
        if tr:
            # (hi + lo) is the exact fp32 value: transpose hi and lo separately is not a valid split of
            # the transposed value only if rounding differed, and tf32 rounding is elementwise
            table = ext.build_transpose_table([(hi, Bc.hi, None, None) for hi, lo, Bc in tr] + [(lo, Bc.lo, None, None) for hi, lo, Bc in tr])
            ext.transpose_split(*table)
            for hi, lo, Bc in tr:
                torch.add(Bc.hi, Bc.lo, out=Bc.plain)
        for s in subs:
            s.A = s.B = None
        return children

    def close_scalar(self, subs: list[Sub]) -> None:
        for s in subs:
            self.lams[s.root][s.offset : s.offset + s.n] = torch.diagonal(s.A.plain)
            cols = self.vecs[s.root][:, s.offset : s.offset + s.n]
            if s.B is None:
                cols.copy_(torch.eye(s.n, device=self.device))
            else:
                cols.copy_(s.B.plain)

    def close_leaves(self, subs: list[Sub]) -> list[int]:
        self._run_leaves(subs, shift=0.0)
        return []  # convergence of the leaves is read once, in finish()

    def _run_leaves(self, subs: list[Sub], shift: float) -> None:
        ext, dev = self.ext, self.device
        direct = [s for s in subs if s.B is None]  # a root that is itself a leaf: eigenvectors as columns
        based = [s for s in subs if s.B is not None]
        lam_of = lambda s: self.lams[s.root][s.offset : s.offset + s.n]  # noqa: E731
        if direct:
            sweeps = ext.jacobi_eigh_into(
                [s.A.plain for s in direct], [self.vecs[s.root] for s in direct], [lam_of(s) for s in direct], False,
                self.jacobi_max_sweeps, self.jacobi_tolerance, shift)
            self._leaf_sweeps.append((direct, sweeps))
        if based:
            holders = _mats(ext, dev, [(s.n, s.n) for s in based])
            sweeps = ext.jacobi_eigh_into(
                [s.A.plain for s in based], [h.plain for h in holders], [lam_of(s) for s in based], True,
                self.jacobi_max_sweeps, self.jacobi_tolerance, shift)
            self._leaf_sweeps.append((based, sweeps))
            table = ext.build_sym_table([(h.plain, h.hi, h.lo, None, 1.0, 0.0) for h in holders])
            ext.shift_scale_split(*table)  # the (hi, lo) pairs of all leaves in one launch
            self._gemm([
                self._spec(s.B, h, None, c=self.vecs[s.root][:, s.offset : s.offset + s.n]) for s, h in zip(based, holders)
            ])

    def finish(self, roots_ok: list[bool]) -> tuple[list[Tensor | None], list[Tensor | None]]:
        roots_ok = list(roots_ok)
        # One-sided Jacobi does not settle on a leaf that is singular or indefinite to working
        # precision (columns of A V that are pure rounding noise): such leaves run once more on
        # A + 1.5 ||A||_F I, which costs them the relative accuracy of their smallest eigenvalues,
        # already lost, and nothing else.
        pending, self._leaf_sweeps = self._leaf_sweeps, []
        stuck = [
            s for subs, sweeps in pending for s, used in zip(subs, sweeps.cpu().tolist(), strict=True)
            if used > self.jacobi_max_sweeps and roots_ok[s.root]
        ]
        if stuck:
            self._run_leaves(stuck, shift=self.jacobi_shift)
            for subs, sweeps in self._leaf_sweeps:
                for s, used in zip(subs, sweeps.cpu().tolist(), strict=True):
                    if used > self.jacobi_max_sweeps:
                        roots_ok[s.root] = False
            self._leaf_sweeps = []
        self.leaves_retried = len(stuck)
        self.failed_in_finish = [i for i, ok in enumerate(roots_ok) if not ok]
        lams: list[Tensor | None] = []
        vecs: list[Tensor | None] = []
        for ok, lam, Q in zip(roots_ok, self.lams, self.vecs, strict=True):
            if not ok:
                lams.append(None)
                vecs.append(None)
                continue
            sorted_lam, order = torch.sort(lam, stable=True)
            lams.append(sorted_lam)
            vecs.append(Q.index_select(1, order))
        return lams, vecs
