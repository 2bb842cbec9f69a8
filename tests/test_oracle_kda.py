"""Pins of the KDA oracle (no GPU): chunked WY form == token recurrence in fp64
at 1e-10 and explicit backward == autodiff at 1e-7, the relations of the
reference's tests/ref/kda/test_naive_kda.py:198-293."""
import pytest
import torch

from oracle import kda as K

DT = torch.float64


def _rand(seed, B, T, H, Kd, V):
    g = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(B, T, H, Kd, dtype=DT, generator=g), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(B, T, H, Kd, dtype=DT, generator=g), dim=-1)
    v = torch.randn(B, T, H, V, dtype=DT, generator=g)
    gate = torch.nn.functional.logsigmoid(torch.randn(B, T, H, Kd, dtype=DT, generator=g))
    beta = torch.sigmoid(torch.randn(B, T, H, dtype=DT, generator=g))
    h0 = torch.randn(B, H, Kd, V, dtype=DT, generator=g)
    return q, k, v, gate, beta, h0


@pytest.mark.parametrize("B,T,H,Kd,V,C", [(2, 64, 2, 16, 24, 16), (1, 70, 2, 32, 16, 32), (1, 1, 1, 8, 8, 16)])
@pytest.mark.parametrize("use_h0", [False, True])
def test_chunk_equals_recurrent(B, T, H, Kd, V, C, use_h0):
    q, k, v, g, beta, h0 = _rand(0, B, T, H, Kd, V)
    h0 = h0 if use_h0 else None
    o1, s1 = K.naive_recurrent_kda(q, k, v, g, beta, None, h0, True)
    o2, s2 = K.naive_chunk_kda(q, k, v, g, beta, None, h0, True, chunk_size=C)
    assert (o1 - o2).abs().max() < 1e-10 and (s1 - s2).abs().max() < 1e-10


def test_explicit_backward_equals_autodiff():
    q, k, v, g, beta, h0 = _rand(1, 2, 40, 2, 16, 24)
    leaves = [x.clone().requires_grad_() for x in (q, k, v, g, beta, h0)]
    o, s = K.naive_recurrent_kda(*leaves[:5], None, leaves[5], True)
    do, dht = torch.randn_like(o), torch.randn_like(s)
    ((o * do).sum() + (s * dht).sum()).backward()
    got = K.fused_recurrent_kda_bwd(q, k, v, g, beta, do, None, h0, dht)
    for a, b in zip(got, leaves):
        assert (a - b.grad).abs().max() < 1e-7
    # gradients of the chunked form agree too
    leaves2 = [x.clone().requires_grad_() for x in (q, k, v, g, beta, h0)]
    o2, s2 = K.naive_chunk_kda(*leaves2[:5], None, leaves2[5], True, chunk_size=16)
    ((o2 * do).sum() + (s2 * dht).sum()).backward()
    for a, b in zip(leaves2, leaves):
        assert (a.grad - b.grad).abs().max() < 1e-7


@pytest.mark.parametrize("B,T,H,Kd,V,C", [(2, 64, 2, 16, 24, 16), (1, 128, 2, 32, 16, 64), (1, 64, 3, 8, 8, 32)])
@pytest.mark.parametrize("use_h0", [False, True])
def test_staged_chunk_forward_equals_recurrent(B, T, H, Kd, V, C, use_h0):
    """chunk_kda_fwd (cumsum -> Aqk / Akk^-1 -> w, u -> delta-rule scan -> output) against the token
    recurrence: one convention for Akk ((I + stril(beta k k^T 2^dG))^-1, beta on the right-hand
    sides), pinned end to end (fp64, 1e-10)."""
    q, k, v, g, beta, h0 = _rand(2, B, T, H, Kd, V)
    h0 = h0 if use_h0 else None
    o1, s1 = K.naive_recurrent_kda(q, k, v, g, beta, None, h0, True)
    o2, s2, gcs, Aqk, Akk = K.chunk_kda_fwd(q, k, v, g, beta, None, h0, True, chunk_size=C)
    assert (o1 - o2).abs().max() < 1e-10 and (s1 - s2).abs().max() < 1e-10
    assert gcs.shape == g.shape and Aqk.shape == (B, T, H, C) and Akk.shape == (B, T, H, C)
    # Akk is unit lower triangular; Aqk is lower triangular with the diagonal
    A = Akk.reshape(B, T // C, C, H, C)
    i = torch.arange(C)
    assert (A[:, :, i, :, i] - 1).abs().max() < 1e-12
    assert torch.triu(A.permute(0, 1, 3, 2, 4), 1).abs().max() == 0
    assert torch.triu(Aqk.reshape(B, T // C, C, H, C).permute(0, 1, 3, 2, 4), 1).abs().max() == 0


@pytest.mark.parametrize("B,T,H,Kd,V,C", [(2, 64, 2, 16, 24, 16), (1, 128, 2, 32, 16, 64)])
@pytest.mark.parametrize("use_h0", [False, True])
def test_staged_chunk_backward_equals_autodiff(B, T, H, Kd, V, C, use_h0):
    """The six-stage chunk backward (dAv, dhu, fused WY, intra, reverse cumsum, 1/ln2) against autodiff
    of the token recurrence and against the explicit token-level backward (fp64, 1e-7), as
    tests/ref/kda/test_naive_kda.py:198-293 does for the reference."""
    q, k, v, g, beta, h0 = _rand(3, B, T, H, Kd, V)
    h0 = h0 if use_h0 else None
    gen = torch.Generator().manual_seed(9)
    do = torch.randn(B, T, H, V, dtype=DT, generator=gen)
    dht = torch.randn(B, H, Kd, V, dtype=DT, generator=gen)
    names = ("q", "k", "v", "g", "beta") + (("h0",) if use_h0 else ())
    leaves = [x.clone().requires_grad_() for x in (q, k, v, g, beta)] + ([h0.clone().requires_grad_()] if use_h0 else [])
    o, s = K.naive_recurrent_kda(*leaves[:5], None, leaves[5] if use_h0 else None, True)
    ((o * do).sum() + (s * dht).sum()).backward()
    o2, ht2, dq, dk, dv, dg, db, dh0 = K.chunk_kda_with_grads(q, k, v, g, beta, do, None, h0, dht, chunk_size=C)
    assert (o2 - o).abs().max() < 1e-10 and (ht2 - s).abs().max() < 1e-10
    got = dict(q=dq, k=dk, v=dv, g=dg, beta=db, h0=dh0)
    for n, leaf in zip(names, leaves):
        assert (got[n] - leaf.grad).abs().max() < 1e-7, n
    if not use_h0:
        assert dh0 is None
    exp = K.fused_recurrent_kda_bwd(q, k, v, g, beta, do, None, h0, dht)
    for a, b in zip((dq, dk, dv, dg, db), exp):
        assert (a - b).abs().max() < 1e-7


def test_chunk_matrices_against_a_literal_construction():
    """Aqk and Akk of `kda_intra_chunk_fwd` against loops over (i, j) and a general linear solve — the way the
    reference's own test builds them (tests/ops/kda/test_chunk_kda_bwd_tpu.py:56-97), with the convention of the
    accelerator kernel: Akk = (I + stril(beta_i k_i.k_j 2^(G_i - G_j)))^-1 (tops/ops/kda/chunk_intra.py:141-153)."""
    B, T, H, Kd, C = 1, 16, 2, 8, 8
    q, k, _, gate, beta, _ = _rand(11, B, T, H, Kd, 8)
    scale = Kd ** -0.5
    g2 = K.kda_gate_chunk_cumsum(gate, C)          # chunk-local cumulative gate in log2 space
    Aqk, Akk = K.kda_intra_chunk_fwd(q, k, g2, beta, scale, C)
    for h in range(H):
        for c0 in range(0, T, C):
            Lm = torch.zeros(C, C, dtype=DT)
            Am = torch.zeros(C, C, dtype=DT)
            for i in range(C):
                for j in range(i + 1):
                    w = torch.exp2(g2[0, c0 + i, h] - g2[0, c0 + j, h])
                    Am[i, j] = scale * (q[0, c0 + i, h] * k[0, c0 + j, h] * w).sum()
                    if j < i:
                        Lm[i, j] = beta[0, c0 + i, h] * (k[0, c0 + i, h] * k[0, c0 + j, h] * w).sum()
            inv = torch.linalg.solve(torch.eye(C, dtype=DT) + Lm, torch.eye(C, dtype=DT))
            assert (Aqk[0, c0:c0 + C, h] - Am).abs().max() < 1e-12
            assert (Akk[0, c0:c0 + C, h] - inv).abs().max() < 1e-12


# --- the intra-chunk backward on its own: the properties the reference checks in
# tests/ref/kda/test_chunk_kda.py:180-397 (zero cotangents, beta = 0, chunks of one token, linearity),
# and, beyond them, equality with autodiff of the two matrices' definitions ---

def _intra_inputs(seed, B, NT, H, C, Kd):
    gen = torch.Generator().manual_seed(seed)
    T = NT * C
    q = torch.randn(B, T, H, Kd, dtype=DT, generator=gen)
    k = torch.randn(B, T, H, Kd, dtype=DT, generator=gen)
    raw = torch.nn.functional.logsigmoid(torch.randn(B, T, H, Kd, dtype=DT, generator=gen))
    g = raw.reshape(B, NT, C, H, Kd).cumsum(2).reshape(B, T, H, Kd)
    beta = torch.sigmoid(torch.randn(B, T, H, dtype=DT, generator=gen))
    lower = torch.tril(torch.ones(C, C, dtype=torch.bool))[None, None, :, None, :]
    strict = torch.tril(torch.ones(C, C, dtype=torch.bool), -1)[None, None, :, None, :]
    dAqk = torch.where(lower, torch.randn(B, NT, C, H, C, dtype=DT, generator=gen), 0.0).reshape(B, T, H, C)
    dAkk = torch.where(strict, torch.randn(B, NT, C, H, C, dtype=DT, generator=gen), 0.0).reshape(B, T, H, C)
    return q, k, g, beta, dAqk, dAkk


def _intra(q, k, g, beta, dAqk, dAkk, C):
    z = torch.zeros_like(q)
    return K.chunk_kda_bwd_intra(q, k, g, beta, dAqk, dAkk, z, z.clone(), torch.zeros_like(beta), z.clone(), C)


INTRA_SHAPES = [(2, 2, 4, 16, 32), (1, 4, 2, 16, 16), (2, 1, 4, 32, 16), (1, 1, 1, 4, 1), (1, 2, 1, 2, 8),
                (1, 3, 2, 16, 32), (1, 2, 2, 64, 32)]


@pytest.mark.parametrize("B,NT,H,C,Kd", INTRA_SHAPES)
def test_intra_backward_zero_cotangents(B, NT, H, C, Kd):
    q, k, g, beta, dAqk, dAkk = _intra_inputs(42, B, NT, H, C, Kd)
    dq, dk, db, dg = _intra(q, k, g, beta, dAqk, torch.zeros_like(dAkk), C)
    assert dq.shape == q.shape and dk.shape == k.shape and db.shape == beta.shape and dg.shape == g.shape
    assert dq.abs().max() > 0 and db.abs().max() <= 1e-15
    dq2, _, db2, _ = _intra(q, k, g, beta, torch.zeros_like(dAqk), dAkk, C)
    assert dq2.abs().max() <= 1e-15
    if C > 1 and dAkk.abs().max() > 0:
        assert db2.abs().max() > 0


def test_intra_backward_beta_zero_and_single_token_chunks():
    q, k, g, _, dAqk, dAkk = _intra_inputs(55, 1, 2, 2, 8, 4)
    beta0 = torch.zeros(1, 16, 2, dtype=DT)
    dq, dk, db, _ = _intra(q, k, g, beta0, torch.zeros_like(dAqk), dAkk, 8)
    assert dq.abs().max() <= 1e-15 and dk.abs().max() <= 1e-15 and db.abs().max() > 0
    # chunks of one token: the strictly lower triangle is empty
    q, k, g, beta, dAqk, dAkk = _intra_inputs(33, 1, 8, 2, 1, 4)
    assert dAkk.abs().max() == 0
    dq, _, db, _ = _intra(q, k, g, beta, dAqk, dAkk, 1)
    assert dq.abs().max() > 0 and db.abs().max() <= 1e-15


def test_intra_backward_is_linear_in_its_cotangents():
    q, k, g, beta, dAqk, dAkk = _intra_inputs(88, 1, 2, 2, 8, 4)
    zq, zk = torch.zeros_like(dAqk), torch.zeros_like(dAkk)
    one = _intra(q, k, g, beta, dAqk, zk, 8)
    pi = _intra(q, k, g, beta, 3.14 * dAqk, zk, 8)
    for a, b in zip(one, pi):
        assert (b - 3.14 * a).abs().max() <= 1e-10 * (1 + a.abs().max())
    one = _intra(q, k, g, beta, zq, dAkk, 8)
    e = _intra(q, k, g, beta, zq, 2.71 * dAkk, 8)
    for a, b in zip(one, e):
        assert (b - 2.71 * a).abs().max() <= 1e-10 * (1 + a.abs().max())
    both = _intra(q, k, g, beta, dAqk, dAkk, 8)
    parts = _intra(q, k, g, beta, dAqk, zk, 8)
    for a, b, c in zip(both, parts, one):
        assert (a - b - c).abs().max() <= 1e-10 * (1 + a.abs().max())


@pytest.mark.parametrize("B,NT,H,C,Kd", [(1, 2, 2, 8, 4), (2, 3, 1, 16, 8)])
def test_intra_backward_equals_autodiff_of_the_definitions(B, NT, H, C, Kd):
    """dq, dk, dbeta and the gate gradient (before its reverse cumsum: with respect to the cumulative
    gate in log2 space, times ln 2 folded as the stage formulas do) against torch autograd through
    Aqk[i,j] = sum_k q_i k_j 2^(G_i - G_j) (j <= i), Lkk[i,j] = beta_i sum_k k_i k_j 2^(G_i - G_j) (j < i)."""
    q, k, g, beta, dAqk, dAkk = _intra_inputs(7, B, NT, H, C, Kd)
    qa, ka, ga, ba = (x.clone().requires_grad_(True) for x in (q, k, g, beta))
    ch = lambda x: x.reshape(B, NT, C, H, -1)
    qc, kc, gc, bc = ch(qa), ch(ka), ch(ga), ba.reshape(B, NT, C, H)
    dec = torch.exp2(gc[:, :, :, None] - gc[:, :, None, :])                          # [B,NT,i,j,H,K]
    qk = torch.einsum("bnihk,bnijhk,bnjhk->bnihj", qc, dec, kc)
    kk = torch.einsum("bnihk,bnijhk,bnjhk->bnihj", kc, dec, kc) * bc[..., None]
    loss = (qk * ch(dAqk)).sum() + (kk * ch(dAkk)).sum()       # the cotangents are masked already
    loss.backward()
    dq, dk, db, dg = _intra(q, k, g, beta, dAqk, dAkk, C)
    ln2 = 0.6931471805599453
    for name, got, want in (("dq", dq, qa.grad), ("dk", dk, ka.grad), ("db", db, ba.grad), ("dg", dg, ga.grad / ln2)):
        assert (got - want).abs().max() <= 1e-10 * (1 + want.abs().max()), name
