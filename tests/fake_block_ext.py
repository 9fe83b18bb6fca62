"""Torch stand-ins for the per-step block kernels, on top of ``fake_ext.FakeExt``.

With these the whole native engine (``optimizers_b200/native_engine.py``) runs on the CPU: block
tables, gradient pointer table, plans of the factor update and of the preconditioner products,
refresh, direction epilogue, all-gather buffers and the gathered apply.  The arithmetic follows
the kernels' formulas (``ops/csrc/block_kernels.cu``) in fp32 torch operations, so the engine's
result can be compared with the torch step of the optimizer; what is tested is the orchestration.

Device addresses become host addresses: the engine hands over raw pointers for the gradients and for
the all-gather slots, and the stand-in turns them back into tensors with ``ctypes``.
"""

import ctypes

import torch

from fake_ext import FakeExt

_DTYPES = {0: torch.float32, 1: torch.bfloat16, 2: torch.float16}


def _at(address, numel, dtype=torch.float32):
    """A 1-D tensor over ``numel`` elements of ``dtype`` that live at host address ``address``."""
    nbytes = numel * torch.empty(0, dtype=dtype).element_size()
    return torch.frombuffer((ctypes.c_char * nbytes).from_address(address), dtype=dtype)


class _Block:
    __slots__ = ("param", "grad_offset", "grad_slot", "m", "n", "n_pad", "m_pad", "m1", "v", "mom", "z", "g_hi", "g_lo",
                 "gt_hi", "gt_lo", "f_hi", "f_lo", "p", "norms", "send", "slot_offset", "ev", "aux")

    def __init__(self, spec):
        for name, value in zip(self.__slots__, spec, strict=True):
            setattr(self, name, value)

    def w(self):
        """The parameter block as an (m, n) view."""
        return self.param if self.param.dim() == 2 else self.param.view(1, -1)

    def state(self, t):
        return None if t is None else t.view(self.m, self.n)


class FakeBlockExt(FakeExt):
    FLAG_SQUARE_ACC, FLAG_PEER_PUSH = 16, 32
    JACOBI_MAX_N = 128

    # -- tables --------------------------------------------------------------------------------
    def build_block_table(self, specs):
        return ([_Block(s) for s in specs], None, len(specs))

    def build_unpack_table(self, specs):
        return (list(specs), None, 0)

    def build_pack_table(self, specs):
        return (list(specs), None, 0)

    def unpack_split(self, specs, _chunks, _n):
        for src, d, hi, lo in specs:
            if src.dim() == 1:
                full = torch.zeros(d, d)
                r, c = torch.triu_indices(d, d)
                full[r, c] = src
                full = full + torch.triu(full, 1).T
            else:
                full = src
            hi[:d, :d].copy_(full)
            if lo is not None:
                lo[:d, :d].zero_()

    def pack_upper(self, specs, _chunks, _n):
        for src, dst in specs:
            d = src.shape[0]
            if dst.dim() == 1:
                r, c = torch.triu_indices(d, d)
                dst.copy_(src[r, c])
            else:
                dst.copy_(src)

    # -- grouped GEMM with the epilogues of the step --------------------------------------------
    def run_gemm_plan(self, specs, _tiles, _n, alpha, beta, split, status, gamma=0.0):
        plain = []
        for spec in specs:
            flags = spec[10]
            if not flags & (self.FLAG_PACKED_C | self.FLAG_SQUARE_ACC):
                plain.append(spec)
                continue
            a_hi, a_lo, b_hi, b_lo, c = spec[:5]
            A = a_hi + (a_lo if a_lo is not None else 0)
            B = b_hi + (b_lo if b_lo is not None else 0)
            acc = (A.double() @ B.double().T).float()
            if flags & self.FLAG_SQUARE_ACC:
                acc = acc * acc
            if flags & self.FLAG_PACKED_C:
                d = acc.shape[0]
                r, col = torch.triu_indices(d, d)
                c.copy_(alpha * acc[r, col] + (beta * c if beta != 0.0 else 0))
            else:
                m, n = acc.shape
                c = c.view(m, n) if c.dim() == 1 else c[:m, :n]  # the state of a 1-D block is 1-D
                c.copy_(alpha * acc + (beta * c if beta != 0.0 else 0))
        if plain:
            super().run_gemm_plan(plain, _tiles, _n, alpha, beta, split, status, gamma)

    # -- the step's pointwise kernels ------------------------------------------------------------
    def grad_prologue(self, blocks, _tiles, _n, grad_ptrs, l2, beta1, beta3, bc1, graft_kind, g_beta2, g_weight, g_bc2,
                      g_eps, write_split, status, num_grad_peers, grad_scale):
        assert num_grad_peers == 0, "the stand-in has no peers"
        pointers = grad_ptrs.tolist()
        for b in blocks:
            w = b.w()
            pitch = w.stride(0)
            span = (b.m - 1) * pitch + b.n
            flat = _at(pointers[b.grad_slot] + 4 * b.grad_offset, span)
            g = torch.as_strided(flat, (b.m, b.n), (pitch, 1)).clone()
            if not bool(torch.isfinite(g).all()):
                status[0] |= 2
            if l2 != 0.0:
                g = g + l2 * w
            if b.g_hi is not None:
                b.g_hi[:, : b.n].copy_(g)
                if b.g_lo is not None:
                    b.g_lo.zero_()
            if b.gt_hi is not None:
                b.gt_hi[:, : b.m].copy_(g.T)
                if b.gt_lo is not None:
                    b.gt_lo.zero_()
            if b.aux == 1:
                continue
            f = g
            m1 = b.state(b.m1)
            if m1 is not None:
                old = m1.clone()
                m1.copy_(torch.lerp(old, g, 1.0 - beta1))
                f = (torch.lerp(old, g, 1.0 - beta3) if beta3 != beta1 else m1) / bc1
            if b.f_hi is not None:
                b.f_hi[:, : b.n].copy_(f)
                if b.f_lo is not None:
                    b.f_lo.zero_()
            if graft_kind != 0 and b.norms is not None:
                direction = f
                v = b.state(b.v)
                if graft_kind == 2 and v is not None:
                    v.copy_(g_beta2 * v + g_weight * g * g)
                    direction = f / (torch.sqrt(v / g_bc2) + g_eps)
                b.norms[0] += (direction * direction).sum()
            if b.aux == 2:
                b.p.view(b.m, b.n).copy_(f)
                if b.norms is not None:
                    b.norms[1] += (f * f).sum()

    def direction_epilogue(self, blocks, _tiles, _n, lr, graft_only, graft_kind, g_bc2, g_eps, wd_alpha, primal, mu_y, mu_x,
                           classic, momentum, dampening, nesterov, send_dtype, split_input, peer_bases, send_params):
        assert not peer_bases, "the stand-in has no peers"
        lr = float(lr)
        for b in blocks:
            if b.aux == 1:
                continue
            w = b.w()
            if graft_only:
                f = b.f_hi[:, : b.n] + (b.f_lo[:, : b.n] if split_input and b.f_lo is not None else 0)
                v = b.state(b.v)
                d = f / (torch.sqrt(v / g_bc2) + g_eps) if (graft_kind == 2 and v is not None) else f.clone()
            else:
                scale = 1.0
                if graft_kind != 0:
                    scale = torch.sqrt(b.norms[0]) / (torch.sqrt(b.norms[1]) + 1e-16)
                d = b.p.view(b.m, b.n) * scale
            z = b.state(b.z)
            if primal:
                z_old = z * (1.0 - lr * wd_alpha) if wd_alpha != 0.0 else z.clone()
            elif wd_alpha != 0.0:
                d = d + wd_alpha * w
            if classic:
                mom = b.state(b.mom)
                mom.copy_(momentum * mom + (1.0 - dampening) * d)
                d = (1.0 - dampening) * d + momentum * mom if nesterov else mom.clone()
            d = -lr * d
            if primal:
                gap = z_old - w
                z.copy_(z_old + d)
                d = (1.0 - float(mu_x) * float(mu_y)) * d + (1.0 - float(mu_x)) * gap
            if b.send:
                out = d + w if send_params else d
                _at(b.send, b.m * b.n, _DTYPES[send_dtype]).view(b.m, b.n).copy_(out)
            else:
                w.add_(d)

    def _gathered(self, blocks, dtype, update):
        for b in blocks:
            w = b.w()
            d = _at(b.send, b.m * b.n, _DTYPES[dtype]).view(b.m, b.n).float()
            update(b, w, d)

    def gathered_apply(self, blocks, _tiles, _n, dtype, copy_params, status):
        if status is not None and int(status[0]) & 5:
            return
        self._gathered(blocks, dtype, (lambda b, w, d: w.copy_(d)) if copy_params else (lambda b, w, d: w.add_(d)))

    def gathered_apply_scaled(self, blocks, _tiles, _n, dtype, lr, wd_alpha, status):
        if status is not None and int(status[0]) & 5:
            return
        lr = float(lr)
        self._gathered(
            blocks, dtype,
            lambda b, w, d: w.sub_(lr * ((float(b.norms[0]) if b.norms is not None else 1.0) * d + wd_alpha * w)),
        )

    def eig_scale(self, blocks, _tiles, _n, bc2, inv_root, eps, write_split):
        for b in blocks:
            if b.aux == 1:
                continue
            p = b.p.view(b.m, b.n)
            ev = b.ev.view(b.m, b.n)
            b.f_hi[:, : b.n].copy_(p / (torch.pow(ev / bc2, inv_root) + eps))
            if b.f_lo is not None:
                b.f_lo.zero_()

    def mode_switch(self, blocks, _tiles, _n, coeff, send_dtype):
        for b in blocks:
            w, z = b.w(), b.state(b.z)
            delta = coeff * (z - w)
            if b.send:
                _at(b.send, b.m * b.n, _DTYPES[send_dtype]).view(b.m, b.n).copy_(delta)
            else:
                w.add_(delta)

    def peer_barrier(self, *args):
        raise AssertionError("the stand-in has no peers")

    # -- small eigenproblems -------------------------------------------------------------------
    def jacobi_eigh(self, mats, max_sweeps, tol):
        lams, qs = [], []
        for A in mats:
            # the same LAPACK call as the optimizer's torch path: eigenvectors of nearly multiple
            # eigenvalues then agree bit for bit instead of by a rotation inside their subspace
            w, Q = torch.linalg.eigh(A)
            lams.append(w)
            qs.append(Q)
        return lams, qs, torch.full((len(mats),), 3, dtype=torch.int32)
