"""FP64 oracles for the matrix-intra stage (vector-gated intra-chunk interactions).

``matrix_intra_pairwise`` restates the reference's explicit pairwise-gate contraction
(scripts/npu950_intra_regression.py:25-46, ``oracle``); ``matrix_intra_centered`` restates the
centered factorisation the kernels use (tests/test_npu950.py:69-73; kernels/gdn2_consumer_fp32.py:45-60):
with c the per-channel mid-point of the chunk's cumulative gate, alpha = exp2(g-c), zeta = 1/alpha,
  uq = (L (k*zeta))*alpha, ue = (D (k*zeta))*alpha, uk = (L^T (q*alpha) + D^T (k*b*alpha))*zeta.
Gates are chunk-local cumulative values in LOG2 units.  Test infrastructure only.
"""
import numpy as np


def _setup(x, family):
    q, k, g = (x[n].astype(np.float64) for n in ("q", "k", "g"))
    beta = x["beta" if family == "kda" else "b"].astype(np.float64)
    outs = [x[n].astype(np.float64).copy() for n in ("dq", "dk", "db", "dg")]
    return q, k, g, beta, outs


def matrix_intra_pairwise(x, family):
    """x: dict of arrays q,k,g [B,C,H,K]; beta [B,C,H] (kda) or b [B,C,H,K] (gdn2);
    dAqk,dAkk [B,C,H,C]; incoming partial dq,dk,dg [B,C,H,K], db [B,C,H] or [B,C,H,K].
    Returns [dq, dk, db, dg] with the intra contribution added."""
    q, k, g, beta, outs = _setup(x, family)
    B, T, H, K = q.shape
    lower = np.tri(T, dtype=bool)
    for b in range(B):
        for h in range(H):
            gh = g[b, :, h]
            gate = np.exp2(np.where(lower[:, :, None], gh[:, None, :] - gh[None, :, :], 0.0))
            L = np.tril(x["dAqk"][b, :, h].astype(np.float64))
            D = np.tril(x["dAkk"][b, :, h].astype(np.float64), -1)
            be = beta[b, :, h, None] if family == "kda" else beta[b, :, h]
            kk, qq = k[b, :, h], q[b, :, h]
            uq = np.einsum("ij,ijk,jk->ik", L, gate, kk)
            ue = np.einsum("ij,ijk,jk->ik", D, gate, kk)
            uk = np.einsum("ji,jik,jk->ik", L, gate, qq) + np.einsum("ji,jik,jk->ik", D, gate, kk * be)
            outs[0][b, :, h] += uq
            outs[1][b, :, h] += be * ue + uk
            outs[2][b, :, h] += (ue * kk).sum(-1) if family == "kda" else ue * kk
            outs[3][b, :, h] += qq * uq + kk * (be * ue - uk)
    return outs


def matrix_intra_centered(x, family):
    """Same result through the centered matrix form (valid while the per-channel span of g
    over the chunk stays below ~1000 log2 units in FP64)."""
    q, k, g, beta, outs = _setup(x, family)
    B, T, H, K = q.shape
    for b in range(B):
        for h in range(H):
            gh = g[b, :, h]
            c = (gh.max(0) + gh.min(0)) / 2
            alpha, zeta = np.exp2(gh - c), np.exp2(c - gh)
            L = np.tril(x["dAqk"][b, :, h].astype(np.float64))
            D = np.tril(x["dAkk"][b, :, h].astype(np.float64), -1)
            be = beta[b, :, h, None] if family == "kda" else beta[b, :, h]
            kk, qq = k[b, :, h], q[b, :, h]
            uq = (L @ (kk * zeta)) * alpha
            ue = (D @ (kk * zeta)) * alpha
            uk = (L.T @ (qq * alpha) + D.T @ (kk * be * alpha)) * zeta
            outs[0][b, :, h] += uq
            outs[1][b, :, h] += be * ue + uk
            outs[2][b, :, h] += (ue * kk).sum(-1) if family == "kda" else ue * kk
            outs[3][b, :, h] += qq * uq + kk * (be * ue - uk)
    return outs
