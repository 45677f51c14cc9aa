"""Self-checks of the task generators: the group convention, re-derivation of every
target from the input tokens alone, leak-freedom of the tagged formats, and the
degeneracy certificates."""

import itertools

import numpy as np
import pytest

from dual_mod_public_b200.formal import tasks as T

BASE = T.BASE


def test_cayley_convention():
    mul, n = T.cayley("s5")
    perms = sorted(itertools.permutations(range(5)))
    assert n == 120 and mul[0].tolist() == list(range(n)) and mul[:, 0].tolist() == list(range(n))
    rng = np.random.default_rng(0)
    for a, b, c in rng.integers(0, n, size=(200, 3)):
        assert mul[mul[a, b], c] == mul[a, mul[b, c]]
    s01, s12 = perms.index((1, 0, 2, 3, 4)), perms.index((0, 2, 1, 3, 4))
    assert perms[mul[s01, s12]] == (1, 2, 0, 3, 4)           # apply s12 first
    for g, size in (("a5", 60), ("a4xz5", 60), ("z10", 10), ("s3", 6), ("s4", 24)):
        m, k = T.cayley(g)
        assert k == size and sorted(m[3].tolist()) == list(range(k))
    m, k = T.cayley("a4xz5")
    for a, b, c in rng.integers(0, k, size=(100, 3)):
        assert m[m[a, b], c] == m[a, m[b, c]]


def test_group_formats_rederive():
    mul, n = T.cayley("a5")
    rng = T.step_rng(1, 0, 0, 0)
    tok, msk = T.make_group_batch(rng, 4, 10, mul, n)
    g, s = tok[:, 1::2] - BASE, tok[:, 2::2] - BASE - n
    assert (T.running_product(g, mul) == s).all() and msk[:, 2::2].all() and not msk[:, 1::2].any()
    tok, tgt, m2 = T.make_group_tagged_batch(rng, 4, 12, mul, n)
    assert tok.shape == (4, 13) and tok[:, 1:].max() < BASE + n              # states never in the input
    assert (T.running_product(tok[:, 1:] - BASE, mul) == tgt[:, 1:] - BASE - n).all()
    tok, m3, diff = T.make_group_final_batch(rng, 8, 64, mul, n, k_max=6)
    episodes = 0
    for b in range(8):
        p = 1
        while p < 64 and tok[b, p] != 0:
            k = 0
            while tok[b, p + k] != T.QUERY:
                k += 1
            s_ = 0
            for gi in tok[b, p:p + k] - BASE:
                s_ = mul[gi, s_]
            assert tok[b, p + k + 1] == BASE + n + s_ and diff[b, p + k + 1] == k
            p += k + 2
            episodes += 1
    assert episodes > 24


def test_keyed_and_mixed():
    mul, n = T.cayley("a5")
    rng = np.random.default_rng(3)
    K, D = 4, 5
    tok, tgt, msk, depth = T.make_keyed_group_batch(rng, 6, mul, n, K, D, rho=0.25, K_max=8)
    KEYB, ELEMB, STATEB = BASE, BASE + 8, BASE + 8 + n
    for b in range(6):
        state, p = np.zeros(K, dtype=np.int64), 1
        while tok[b, p] != T.QUERY:
            k = tok[b, p] - KEYB
            if tok[b, p + 1] == T.XFROM:
                state[k] = mul[state[k], state[tok[b, p + 2] - KEYB]]
                last = p + 2
            else:
                state[k] = mul[tok[b, p + 1] - ELEMB, state[k]]
                last = p + 1
            assert msk[b, last] and tgt[b, last] == STATEB + state[k]
            p = last + 1
        for _ in range(K):
            assert tgt[b, p + 1] == STATEB + state[tok[b, p + 1] - KEYB] and depth[b, p + 1] == D
            p += 2
    mz, nz = T.cayley("z10")
    tok, tgt, msk, task = T.make_mixed_tagged_batch(rng, 16, 8, mz, nz, mul, n)
    offB = BASE + 2 * nz
    for b in range(16):
        off, mm, nn = (offB, mul, n) if task[b] else (BASE, mz, nz)
        assert (T.running_product(tok[b:b + 1, 1:] - off, mm) == tgt[b:b + 1, 1:] - off - nn).all()


def test_khop_niah_parity_rederive():
    rng = np.random.default_rng(1)
    tok, msk, diff = T.make_khop_batch(rng, 3, 12, 5, 4)
    sym = BASE + 4
    for b in range(3):
        succ = {tok[b, 1 + 3 * i]: tok[b, 3 + 3 * i] for i in range(12)}
        for qi in range(5):
            p = 1 + 36 + 4 * qi
            a = tok[b, p + 1]
            for _ in range(tok[b, p + 2] - BASE + 1):
                a = succ[a]
            assert a == tok[b, p + 3] and msk[b, p + 3] and diff[b, qi] == tok[b, p + 2] - BASE + 1
    tok, msk, diff = T.make_niah_batch(rng, 2, 6, 3, 4)
    assert msk.sum() == 2 * 4 * 3 and diff[msk].max() == 3
    tok, msk = T.make_parity_batch(rng, 4, 9)
    assert ((np.cumsum(tok[:, 1::2] - BASE, axis=1) % 2) == tok[:, 2::2] - BASE - 2).all()


def test_ca_and_match3():
    rng = np.random.default_rng(0)
    tok, tgt, msk = T.make_ca_batch(rng, 8, 16, 5, 110, fmt="silent", pad=3)
    row = tok[:, 3:19] - BASE
    for _ in range(5):
        row = T.CA_RULE[110][4 * np.roll(row, 1, 1) + 2 * row + np.roll(row, -1, 1)]
    assert (tgt[msk].reshape(8, 16) - BASE == row).all()
    for fmt in ("trace", "leaky"):
        t2 = T.make_ca_batch(rng, 2, 8, 4, 90, fmt=fmt, gap=2)
        assert t2[0].shape == t2[1].shape
    marg, short = T.ca_certify(rng, 32, 8, 110, B=512)
    assert T.ca_cell_ok(marg, short)
    rate = T.match3_base_rate(n=20000)
    assert 0.2 < rate < 0.8


def test_matinv_and_dfa():
    rng = np.random.default_rng(0)
    for p in (2, 3):
        for n in (2, 3, 5):
            A, Ai = T.gl_sample(rng, 64, n, p)
            eye = np.broadcast_to(np.eye(n, dtype=np.int64), (64, n, n))
            assert (((A @ Ai) % p) == eye).all()
            tok, tgt, msk = T.make_matinv_batch(rng, 16, n, p, "solve")
            Ab = (tok[:, 3:3 + n * n] - BASE).reshape(16, n, n)
            b = tok[:, 3 + n * n:3 + n * n + n] - BASE
            x = tgt[msk].reshape(16, n) - BASE
            assert (((Ab @ x[:, :, None]) % p).reshape(16, n) == b).all()
    marg, ident = T.mi_certify(rng, 4, 2, "inv", B=512)
    assert marg < 0.7
    trans, ns, na, crasp = T.dfa_lib("contains_ab")
    tok, tgt, msk = T.make_dfa_batch(rng, 4, 20, trans, ns, na, sep=True)
    assert tok.shape == (4, 42) and msk[:, 1::2].all() and crasp
    q = np.zeros(4, dtype=np.int64)
    for t in range(20):
        q = trans[q, tok[:, 2 + 2 * t] - BASE]
        assert (tgt[:, 3 + 2 * t] == BASE + na + q).all()
    assert T.dfa_lib("a5")[1] == 60 and not T.dfa_lib("flipflop")[3]


def test_cvp():
    rng = np.random.default_rng(0)
    tok, tgt, msk, depth = T.make_cvp_batch(rng, 4, 16, m=8, fmt="tagged", chain=1.0)
    assert msk.sum() == 4 * 20 and depth[msk].max() == 16
    vals, _ = T.cvp_values_from_tokens(tok, 8, 16)
    assert (tgt[msk].reshape(4, -1)[:, :16] - (BASE + 24 + 2) == vals[:, 8:]).all()
    t2 = T.make_cvp_batch(rng, 4, 16, m=8, fmt="silent", pad=5, chain=0.0)
    assert t2[0].shape[1] == 1 + 16 + 80 + 5 + 8 and t2[2].sum() == 16
    t3 = T.make_cvp_batch(rng, 4, 16, m=8, fmt="tagged", leak_every=4)
    assert t3[0].shape[1] == 1 + 16 + 80 + 4 + 8
    t4 = T.make_cvp_batch(rng, 6, 16, m=8, n_topo=3, addr="rel")
    assert t4[0].shape[0] == 6
    marg, short = T.cvp_certify(np.random.default_rng(1), 32, m=16, B=1024, n_batches=3)
    assert T.cvp_cell_ok(marg, short)
