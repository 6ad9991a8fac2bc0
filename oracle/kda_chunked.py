"""Chunked WY restatement of KDA with a hand-written backward (CPU, PyTorch).

TEST INFRASTRUCTURE ONLY (see kda_oracle.py).  This module restates, chunk by
chunk, the algebra the reference's production kernels implement
(nanochat/mixers/cuda_kda/chunk_wy_forward.cu:125-405, 761-858, 940-1275,
1498-1588 for the forward; chunk_wy_backward.cu:2445-2562, 2818-3331,
3337-3552, 3787-3894 for the backward) so that every intermediate of the CUDA
kernels (A, M, T, U, W, Z, H and their adjoints) can be compared one by one.
It is validated against autograd through the token recurrence in
tests/test_oracle_chunked.py.

Per chunk of C tokens of one (sequence, head), H = incoming state [K,V]:
  G = cumsum(g)                       (per channel, within the chunk)
  A[i,s] = sum_d qn[i,d] kn[s,d] exp(G[i,d]-G[s,d]),  s <= i
  M[i,s] = beta_i sum_d kn[i,d] kn[s,d] exp(G[i,d]-G[s,d]),  s < i
  T = (I + M)^-1 ;  U = T (beta*v) ;  W = T (beta*exp(G)*kn)
  Z = U - W H ;  O = (qn*exp(G)) H + A Z
  H' = exp(G_end) * H + (kn*exp(G_end-G))^T Z
"""

from __future__ import annotations

from typing import Optional

import torch

Tensor = torch.Tensor


def _norm_fwd(x, eps=1e-12):
    n = x.norm(dim=-1, keepdim=True).clamp_min(eps)
    return x / n, 1.0 / n


def chunk_forward_single(q, k, v, g, beta, h0, scale, C=64, l2norm=True):
    """One (sequence, head).  q,k,g [T,K]; v [T,V]; beta [T]; h0 [K,V].

    Returns o [T,V], final state [K,V] and the per-chunk records used by the
    backward.
    """
    T, K = q.shape
    dt = q.dtype
    if l2norm:
        qh, qinv = _norm_fwd(q)
        kh, kinv = _norm_fwd(k)
    else:
        qh, kh = q, k
        qinv = kinv = torch.ones(T, 1, dtype=dt)
    qn = qh * scale
    kn = kh
    H = h0.clone()
    o = torch.empty(T, v.shape[1], dtype=dt)
    recs = []
    for c0 in range(0, T, C):
        c1 = min(T, c0 + C)
        L = c1 - c0
        qc, kc, vc, gc, bc = qn[c0:c1], kn[c0:c1], v[c0:c1], g[c0:c1], beta[c0:c1]
        G = torch.cumsum(gc, dim=0)                       # [L,K]
        rho = torch.exp(G[:, None, :] - G[None, :, :])    # [i,s,d], used only for s<=i
        low = torch.tril(torch.ones(L, L, dtype=dt))
        slow = torch.tril(torch.ones(L, L, dtype=dt), -1)
        rho = rho * low[:, :, None]                       # avoid inf*0 above the diagonal
        A = torch.einsum("id,sd,isd->is", qc, kc, rho) * low
        Mt = torch.einsum("id,sd,isd->is", kc, kc, rho) * slow   # without beta
        M = bc[:, None] * Mt
        Tm = torch.linalg.solve_triangular(torch.eye(L, dtype=dt) + M, torch.eye(L, dtype=dt), upper=False)
        eG = torch.exp(G)
        P = bc[:, None] * vc
        Q = bc[:, None] * eG * kc
        U = Tm @ P
        W = Tm @ Q
        Z = U - W @ H
        R = qc * eG
        o[c0:c1] = R @ H + A @ Z
        Gend = G[-1]
        E = kc * torch.exp(Gend[None, :] - G)
        recs.append(dict(c0=c0, c1=c1, G=G, A=A, Mt=Mt, T=Tm, P=P, Q=Q, U=U, W=W, Z=Z, R=R, E=E, H=H.clone()))
        H = torch.exp(Gend)[:, None] * H + E.t() @ Z
    aux = dict(qn=qn, kn=kn, qinv=qinv, kinv=kinv, recs=recs, scale=scale, l2norm=l2norm)
    return o, H, aux


def chunk_backward_single(q, k, v, g, beta, aux, do, dhT):
    """Hand-derived VJP.  do [T,V]; dhT [K,V] cotangent of the final state (or None).

    Returns dq, dk, dv, dg, dbeta, dh0.
    """
    T, K = q.shape
    V = v.shape[1]
    dt = q.dtype
    qn, kn = aux["qn"], aux["kn"]
    dqn = torch.zeros(T, K, dtype=dt)
    dkn = torch.zeros(T, K, dtype=dt)
    dv = torch.zeros(T, V, dtype=dt)
    dg = torch.zeros(T, K, dtype=dt)
    dbeta = torch.zeros(T, dtype=dt)
    dHn = torch.zeros(K, V, dtype=dt) if dhT is None else dhT.clone()   # adjoint of the chunk's outgoing state
    for rec in reversed(aux["recs"]):
        c0, c1 = rec["c0"], rec["c1"]
        L = c1 - c0
        G, A, Mt, Tm, P, Q, W, Z, R, E, H = (rec[n] for n in ("G", "A", "Mt", "T", "P", "Q", "W", "Z", "R", "E", "H"))
        qc, kc, vc, bc = qn[c0:c1], kn[c0:c1], v[c0:c1], beta[c0:c1]
        dO = do[c0:c1]
        eG = torch.exp(G)
        Gend = G[-1]
        eGend = torch.exp(Gend)
        low = torch.tril(torch.ones(L, L, dtype=dt))
        slow = torch.tril(torch.ones(L, L, dtype=dt), -1)

        # ---- state-adjoint scan step
        dZ = A.t() @ dO + E @ dHn
        dH = R.t() @ dO + eGend[:, None] * dHn - W.t() @ dZ
        # ---- chunk-local products
        dR = dO @ H.t()
        dE = Z @ dHn.t()
        dWm = dZ @ H.t()                      # enters with a minus sign (Z = U - W H)
        dq_c = dR * eG
        dk_c = dE * torch.exp(Gend[None, :] - G)
        dG = dR * R - dE * E
        dGend = (dE * E).sum(dim=0) + eGend * (dHn * H).sum(dim=1)
        dP = Tm.t() @ dZ
        dv[c0:c1] = bc[:, None] * dP
        db = (dP * vc).sum(dim=1)
        dQ = -(Tm.t() @ dWm)
        dk_c = dk_c + dQ * bc[:, None] * eG
        dG = dG + dQ * bc[:, None] * eG * kc
        db = db + (dQ * eG * kc).sum(dim=1)
        X = dZ @ P.t() - dWm @ Q.t()          # adjoint of T
        dM = -(Tm.t() @ X @ Tm.t()) * slow
        dA = (dO @ Z.t()) * low
        # ---- pull A and M back to qn, kn, G, beta
        rho = torch.exp(G[:, None, :] - G[None, :, :]) * low[:, :, None]
        a = dA[:, :, None] * rho                          # [i,s,d]
        m = (bc[:, None] * dM)[:, :, None] * rho
        dq_c = dq_c + torch.einsum("isd,sd->id", a, kc)
        dk_c = dk_c + torch.einsum("isd,id->sd", a, qc) + torch.einsum("isd,id->sd", m, kc) \
                    + torch.einsum("isd,sd->id", m, kc)
        summand = a * qc[:, None, :] * kc[None, :, :] + m * kc[:, None, :] * kc[None, :, :]
        dG = dG + summand.sum(dim=1) - summand.sum(dim=0)
        db = db + (dM * Mt).sum(dim=1)
        dG[-1] = dG[-1] + dGend
        dg[c0:c1] = torch.flip(torch.cumsum(torch.flip(dG, [0]), dim=0), [0])
        dqn[c0:c1] = dq_c
        dkn[c0:c1] = dk_c
        dbeta[c0:c1] = db
        dHn = dH
    sc = aux["scale"]
    if aux["l2norm"]:
        qh = qn / sc
        dqh = dqn * sc
        dq = aux["qinv"] * (dqh - qh * (qh * dqh).sum(dim=-1, keepdim=True))
        dk = aux["kinv"] * (dkn - kn * (kn * dkn).sum(dim=-1, keepdim=True))
    else:
        dq, dk = dqn * sc, dkn
    return dq, dk, dv, dg, dbeta, dHn


def chunk_kda(q, k, v, g, beta, *, initial_state: Optional[Tensor] = None, scale=None, C=64, l2norm=True):
    """Batched driver over [B,T,H,*]; returns (o, final_state V-first, aux list)."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    sc = K ** -0.5 if scale is None else scale
    o = torch.empty(B, T, H, V, dtype=q.dtype)
    fs = torch.empty(B, H, V, K, dtype=q.dtype)
    auxes = {}
    for b in range(B):
        for h in range(H):
            h0 = torch.zeros(K, V, dtype=q.dtype) if initial_state is None else initial_state[b, h].t().to(q.dtype)
            oo, hT, aux = chunk_forward_single(q[b, :, h], k[b, :, h], v[b, :, h], g[b, :, h], beta[b, :, h], h0, sc, C, l2norm)
            o[b, :, h] = oo
            fs[b, h] = hT.t()
            auxes[(b, h)] = aux
    return o, fs, auxes


def chunk_kda_backward(q, k, v, g, beta, auxes, do, dfs=None):
    B, T, H, K = q.shape
    dq = torch.empty_like(q); dk = torch.empty_like(k); dv = torch.empty_like(v)
    dg = torch.empty_like(g); db = torch.empty_like(beta)
    dh0 = torch.empty(B, H, v.shape[-1], K, dtype=q.dtype)
    for b in range(B):
        for h in range(H):
            dhT = None if dfs is None else dfs[b, h].t().to(q.dtype)
            r = chunk_backward_single(q[b, :, h], k[b, :, h], v[b, :, h], g[b, :, h], beta[b, :, h],
                                      auxes[(b, h)], do[b, :, h], dhT)
            dq[b, :, h], dk[b, :, h], dv[b, :, h], dg[b, :, h], db[b, :, h] = r[:5]
            dh0[b, h] = r[5].t()
    return dq, dk, dv, dg, db, dh0
