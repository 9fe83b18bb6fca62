"""A torch stand-in for the CUDA extension, for CPU tests of the host logic that drives it.

``FakeExt`` implements the calls that ``optimizers_b200/matrix/batched.py`` and the native backend
of ``optimizers_b200/matrix/eigh_dc.py`` make (launch tables, grouped products with their epilogue
flags and operand views, the per-matrix passes, the Householder factorisation, the Jacobi leaves)
with plain torch on whatever device the tensors live on.  Products are formed in fp64 and rounded
once, operand pairs are (value, 0): the arithmetic is at least as accurate as the kernels', so a
test that passes here checks the Python around the kernels, not the kernels.
"""

import torch


class FakeExt:
    FLAG_PACKED_C, FLAG_SPLIT_OUT, FLAG_SUMSQ, FLAG_NO_C = 1, 2, 4, 8
    FLAG_MIRROR, FLAG_ADD_DIAG, FLAG_TRACE = 64, 128, 256

    def __init__(self):
        self.gemm_launches = 0
        self.calls = []

    # -- scratch matrices ------------------------------------------------------------------------
    def alloc_mat_batch(self, rows, cols, plain, pair, device):
        count = int(plain) + 2 * int(pair)
        pitch = [(c + 3) // 4 * 4 for c in cols]
        block = torch.full((max(sum(count * r * ld for r, ld in zip(rows, pitch)), 1),), float("nan"), device=device)
        out, offset = [], 0
        for r, c, ld in zip(rows, cols, pitch):
            views = [None, None, None]
            for k in range(3):
                if plain if k == 0 else pair:
                    views[k] = torch.as_strided(block, (r, c), (ld, 1), offset)
                    offset += r * ld
            out.append(tuple(views))
        return out

    # -- operand split -------------------------------------------------------------------------
    def tf32_split(self, src, hi, lo):
        hi.copy_(src)
        lo.zero_()

    # -- grouped GEMM --------------------------------------------------------------------------
    def build_gemm_plan(self, specs):
        return (list(specs), None, 0)

    def run_gemm_plan(self, specs, _tiles, _n, alpha, beta, split, status, gamma=0.0):
        self.gemm_launches += 1
        self.calls.append("grouped_gemm")
        for spec in specs:
            a_hi, a_lo, b_hi, b_lo, c, d_hi, d_lo, sumsq, _ldc, _ldd, flags, upper = spec[:12]
            A = a_hi + (a_lo if a_lo is not None else 0)
            B = b_hi + (b_lo if b_lo is not None else 0)
            if len(spec) == 14 and spec[13] is not None:
                ar, ak, br, bk, M, N, K = spec[13]
                A, B = A[ar : ar + M, ak : ak + K], B[br : br + N, bk : bk + K]
            assert A.shape[1] == B.shape[1], (A.shape, B.shape)
            out = alpha * (A.double() @ B.double().T).float()
            m, n = out.shape  # outputs may be handed over in their padded storage
            if flags & self.FLAG_MIRROR:
                assert upper and m == n
                out = torch.triu(out) + torch.triu(out, 1).T
            if c is not None and not flags & self.FLAG_NO_C and beta != 0.0:
                out = out + beta * c[:m, :n]
            if flags & self.FLAG_ADD_DIAG:
                out = out + gamma * torch.eye(m, n)
            if flags & self.FLAG_SUMSQ:
                sumsq[0] += (out.double() ** 2).sum().float()
            if flags & self.FLAG_TRACE:
                sumsq[1] += torch.trace(out.double()).float()
            if c is not None and not flags & self.FLAG_NO_C:
                c[:m, :n].copy_(out)
            if flags & self.FLAG_SPLIT_OUT:
                d_hi[:m, :n].copy_(out)
                d_lo[:m, :n].zero_()

    # -- coupled iterations ----------------------------------------------------------------------
    def build_mat_table(self, specs):
        return (list(specs), None, 0)

    def affine_identity_split(self, specs, _chunks, _n, a, b):
        for src, hi, lo, _err in specs:
            hi.copy_(a * src + b * torch.eye(src.shape[0]))
            if lo is not None:
                lo.zero_()

    def identity_error(self, specs, _chunks, _n):
        for src, _hi, _lo, err in specs:
            err[0] = (src - torch.eye(src.shape[0])).abs().max()

    # -- per-matrix passes of the eigensolver ------------------------------------------------------
    def build_sym_table(self, specs):
        return (list(specs), None, 0)

    def sym_measure(self, specs, count):
        for src, _hi, _lo, stats, _a, _b in specs[:count]:
            n = src.shape[0]
            mean = torch.trace(src.double()) / n
            stats[0] = mean.float()
            stats[1] = torch.linalg.norm(src.double() - mean * torch.eye(n, dtype=torch.float64)).float()

    def sq_offdiag(self, specs, count):
        for src, _hi, _lo, stats, _a, _b in specs[:count]:
            stats[0] = (src.double() ** 2).sum().float()
            stats[1] = (torch.diagonal(src).double() ** 2).sum().float()

    def shift_scale_split(self, specs, _chunks, _n):
        for src, hi, lo, _stats, a, b in specs:
            n = hi.shape[0]
            value = b * torch.eye(n) if a == 0.0 else a * src + b * torch.eye(n)
            hi.copy_(value)
            if lo is not None:
                lo.zero_()

    def build_transpose_table(self, specs):
        return (list(specs), None, 0)

    def transpose_split(self, specs, _tiles, _n):
        for src, dst, dst_hi, dst_lo in specs:
            if dst is not None:
                dst.copy_(src.T)
            if dst_hi is not None:
                dst_hi.copy_(src.T)
                dst_lo.zero_()

    def householder_qr(self, specs):
        self.calls.append("householder_qr")
        for spec in specs:
            ct, n, k, zt, zt_hi, zt_lo = spec[:6]
            q_rows = spec[6] if len(spec) == 7 else n  # only the first q_rows rows of Q^T are produced
            assert ct.shape == (k, n) and zt.shape[0] >= q_rows
            Q, _ = torch.linalg.qr(ct.T.double(), mode="complete")
            zt[:q_rows].copy_(Q.T.float()[:q_rows])
            if zt_hi is not None:
                zt_hi[:q_rows].copy_(zt[:q_rows])
                zt_lo[:q_rows].zero_()

    def jacobi_eigh_into(self, mats, qs, lams, transposed, max_sweeps, tol, shift_scale):
        for A, q, lam in zip(mats, qs, lams):
            w, Q = torch.linalg.eigh(A.double())
            lam.copy_(w.float())
            q.copy_((Q.T if transposed else Q).float())
        return torch.full((len(mats),), 3, dtype=torch.int32)
