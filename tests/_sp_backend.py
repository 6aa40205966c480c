"""CPU stand-in for the sequence-parallel backend: the per-rank stage math written with torch CPU
ops and the oracle's helpers, with the same `xfer` layouts as the C ABI (see
include/flashnystrom_b200.h, fnb_sp_info).  Test infrastructure only."""
import torch

from oracle import nystrom_oracle as O


class TorchContext:
    def __init__(self, q, k, v, m, J, kappa, rank, world, dtype=torch.float64):
        self.q, self.k, self.v = (t.to(dtype) for t in (q, k, v))       # local shards (B,H,Nl,D)
        B, H, Nl, D = q.shape
        self.B, self.H, self.Nl, self.D, self.m, self.J, self.kappa = B, H, Nl, D, m, J, kappa
        self.BH, self.rank, self.world, self.dtype = B * H, rank, world, dtype
        self.N = world * Nl
        self.seg = self.N // m
        self.s = D ** -0.25
        self.lidx = torch.arange(rank * Nl, (rank + 1) * Nl) // self.seg          # landmark of each local row

    def new_xfer(self, n):
        return torch.zeros(n, dtype=torch.float32)

    # ---- forward -------------------------------------------------------------------------
    def forward_stage(self, stage, x):
        B, H, D, m = self.B, self.H, self.D, self.m
        md, mv = self.BH * m * D, self.BH * m
        if stage == 0:
            sums = torch.zeros(2, B, H, m, D, dtype=self.dtype)
            sums[0].index_add_(2, self.lidx, self.q)
            sums[1].index_add_(2, self.lidx, self.k)
            x[:2 * md] = sums.reshape(-1).float()
        elif stage == 1:
            sums = x[:2 * md].to(self.dtype).view(2, B, H, m, D)
            self.qt, self.kt = sums[0] * (self.s / self.seg), sums[1] * (self.s / self.seg)
            self.K2 = torch.softmax(self.qt @ self.kt.transpose(-2, -1), -1)
            if self.kappa > 0:
                lam = O.ridge_lambda(self.K2, self.kappa)
                self.A = self.K2.transpose(-2, -1) @ self.K2 + lam * torch.eye(m, dtype=self.dtype)
                its = O.newton_schulz(self.A, self.J)
                self.k2inv = its[-1] @ self.K2.transpose(-2, -1)
            else:
                self.A = self.K2
                its = O.newton_schulz(self.A, self.J)
                self.k2inv = its[-1]
            self.iterates = torch.stack(its, dim=2)
            S3 = self.qt @ (self.k * self.s).transpose(-2, -1)                    # (B,H,m,Nl)
            M = S3.max(-1).values
            E = torch.exp(S3 - M[..., None])
            x[:md] = (E @ self.v).reshape(-1).float()
            x[md:md + mv] = M.reshape(-1).float()
            x[md + mv:md + 2 * mv] = E.sum(-1).reshape(-1).float()
        else:
            per = md + 2 * mv
            g = x.to(self.dtype).view(self.world, per)
            acc = g[:, :md].view(self.world, B, H, m, D)
            mx = g[:, md:md + mv].view(self.world, B, H, m)
            sm = g[:, md + mv:].view(self.world, B, H, m)
            M = mx.max(0).values
            wgt = torch.exp(mx - M)
            L = (wgt * sm).sum(0)
            self.bmat = (wgt[..., None] * acc).sum(0) / L[..., None]
            self.lse3 = M + torch.log(L)
            self.step2 = self.k2inv @ self.bmat
            S1 = (self.q * self.s) @ self.kt.transpose(-2, -1)
            self.P1 = torch.softmax(S1, -1)
            self.out = self.P1 @ self.step2

    # ---- backward ------------------------------------------------------------------------
    def begin_backward(self, d_out):
        self.dO = d_out.to(self.dtype)

    def backward_stage(self, stage, x):
        B, H, D, m = self.B, self.H, self.D, self.m
        md = self.BH * m * D
        if stage == 0:
            dP1 = self.dO @ self.step2.transpose(-2, -1)
            self.dS1 = self.P1 * (dP1 - (self.P1 * dP1).sum(-1, keepdim=True))
            part = torch.stack([self.P1.transpose(-2, -1) @ self.dO,
                                self.dS1.transpose(-2, -1) @ (self.q * self.s)], dim=2)   # (B,H,2,m,D)
            x[:2 * md] = part.reshape(-1).float()
        elif stage == 1:
            red = x[:2 * md].to(self.dtype).view(B, H, 2, m, D)
            dstep2, dkt_a = red[:, :, 0], red[:, :, 1]
            dO3 = self.k2inv.transpose(-2, -1) @ dstep2
            G = dstep2 @ self.bmat.transpose(-2, -1)
            D3 = (self.bmat * dO3).sum(-1, keepdim=True)
            if self.kappa > 0:
                ZJ = self.iterates[:, :, -1]
                dA, _ = O.ns_backward(self.A, self.iterates, G @ self.K2)
                dK2 = G.transpose(-2, -1) @ ZJ + self.K2 @ (dA + dA.transpose(-2, -1))
            else:
                dK2, _ = O.ns_backward(self.A, self.iterates, G)
            dS2 = self.K2 * (dK2 - (dK2 * self.K2).sum(-1, keepdim=True))
            self.dqt_ns = dS2 @ self.kt
            dkt_tot = dkt_a + dS2.transpose(-2, -1) @ self.qt
            ks = self.k * self.s
            P3 = torch.exp(self.qt @ ks.transpose(-2, -1) - self.lse3[..., None])        # (B,H,m,Nl)
            dS3 = P3 * (dO3 @ self.v.transpose(-2, -1) - D3)
            self.dv = P3.transpose(-2, -1) @ dO3
            self.dk = self.s * (dS3.transpose(-2, -1) @ self.qt + (dkt_tot / self.seg)[:, :, self.lidx])
            x[:md] = (dS3 @ ks).reshape(-1).float()
        else:
            dqt_tot = self.dqt_ns + x[:md].to(self.dtype).view(B, H, m, D)
            self.dq = self.s * (self.dS1 @ self.kt + (dqt_tot / self.seg)[:, :, self.lidx])
