"""On-the-fly generators of the formal-language / state-tracking tasks.

Every task yields fresh numpy batches from a seeded generator: there is no corpus
and nothing to memorise.  Token layout (shared by all tasks, so checkpoints stay
interchangeable with the reference harness): 0 PAD, 1 BOS, 2 ARROW, 3 QUERY,
4 XFROM / SEP, 5-7 reserved, task tokens from 8.  Targets always live in a token
range disjoint from the inputs.  "Tagged" tasks return (tok, tgt, msk): the loss
at a position compares the logits AT that position with tgt (not next-token);
the older interleaved formats return (tok, msk) for next-token loss.

Group convention: permutations are tuples p with p[i] = p(i); (a @ b)(x) =
a(b(x)); MUL[a, b] = index(a @ b); the running state after op g_i is
s_i = MUL[g_i, s_{i-1}], identity = index 0.

Tasks: group (z*, s3, s4, s5, a5, a4xz5) in interleaved / tagged / final formats,
mixed two-group rows, keyed group accumulation, k-hop pointer chasing, multi-token
key-value recall, parity, elementary cellular automata (rule 90 / 110) with a
degeneracy certificate, match-3, GF(p) matrix inverse / solve / product, DFA state
prediction and the keyed XOR-majority circuit value problem with its certificate.
`step_rng(task, seed, split, step)` gives the byte-identical stream per seed.

Reference parity: formal_language/harness/statetrack_gen.py (cayley 49-84, group
formats 87-169, keyed 172-255, mixed 258-285, khop 289-327, niah 330-367, parity
371-382, CA 386-480, match3 484-536, step_rng 541-542, matinv 647-760, dfa
763-827, cvp 830-1006).
"""

from __future__ import annotations

import itertools

import numpy as np

PAD, BOS, ARROW, QUERY, XFROM = 0, 1, 2, 3, 4
SEP = 4
BASE = 8


def step_rng(task_id, seed, split, step):
    return np.random.default_rng([task_id, seed, split, step])


def _blank(B, T, n_side=0):
    """(tok with BOS set, n_side zeroed int64 side arrays..., bool mask), all [B, T]."""
    tok = np.zeros((B, T), dtype=np.int64)
    tok[:, 0] = BOS
    side = [np.zeros((B, T), dtype=np.int64) for _ in range(n_side)]
    return (tok, *side, np.zeros((B, T), dtype=bool))


# ============================================================================== groups
def _is_even(p):
    return sum(p[i] > p[j] for i in range(len(p)) for j in range(i + 1, len(p))) % 2 == 0


def _perm_table(perms):
    index = {p: i for i, p in enumerate(perms)}
    k = len(perms[0])
    n = len(perms)
    mul = np.empty((n, n), dtype=np.int16)
    for i, a in enumerate(perms):
        for j, b in enumerate(perms):
            mul[i, j] = index[tuple(a[b[x]] for x in range(k))]
    return mul, n


def cayley(group):
    """(MUL [n, n] int16, n) for z<m>, s3, s4, s5, a5 or a4xz5 (A4 x Z5: solvable,
    non-abelian, 60 elements like A5)."""
    if group.startswith("z"):
        m = int(group[1:])
        r = np.arange(m)
        return ((r[:, None] + r[None, :]) % m).astype(np.int16), m
    if group == "a4xz5":
        mul4, n4 = _perm_table(sorted(p for p in itertools.permutations(range(4)) if _is_even(p)))
        i = np.arange(n4 * 5)
        pa, za = i // 5, i % 5
        mul = mul4[pa[:, None], pa[None, :]].astype(np.int64) * 5 + (za[:, None] + za[None, :]) % 5
        return mul.astype(np.int16), n4 * 5
    if group == "a5":
        return _perm_table(sorted(p for p in itertools.permutations(range(5)) if _is_even(p)))
    k = {"s3": 3, "s4": 4, "s5": 5}[group]
    return _perm_table(sorted(itertools.permutations(range(k))))


def running_product(g, mul):
    """s[:, t] = MUL[g[:, t], s[:, t-1]] from the identity; g [B, n]."""
    s = np.empty_like(g, dtype=np.int64)
    prev = np.zeros(g.shape[0], dtype=np.int64)
    for t in range(g.shape[1]):
        prev = mul[g[:, t], prev].astype(np.int64)
        s[:, t] = prev
    return s


def make_group_batch(rng, B, n_ops, mul, n):
    """Interleaved [BOS, g1, s1, g2, s2, ...]; next-token loss at the state slots."""
    g = rng.integers(0, n, size=(B, n_ops))
    s = running_product(g, mul)
    tok, msk = _blank(B, 1 + 2 * n_ops)
    tok[:, 1::2], tok[:, 2::2] = BASE + g, BASE + n + s
    msk[:, 2::2] = True
    return tok, msk


def make_group_tagged_batch(rng, B, n_ops, mul, n, op_pool=None):
    """Ops-only input [BOS, g1..gN]; at the position of g_i the target is the running
    product s_i (states never appear in the input)."""
    if op_pool is None:
        g = rng.integers(0, n, size=(B, n_ops))
    else:
        g = np.asarray(op_pool)[rng.integers(0, len(op_pool), size=(B, n_ops))]
    s = running_product(g, mul)
    tok, tgt, msk = _blank(B, 1 + n_ops, 1)
    tok[:, 1:], tgt[:, 1:], msk[:, 1:] = BASE + g, BASE + n + s, True
    return tok, tgt, msk


def make_group_final_batch(rng, B, T, mul, n, k_max, k_min=1):
    """Rows packed with independent episodes [g x k, QUERY, s_k]; loss at s_k only.
    Returns (tok, msk, diff) with diff = k at the scored positions."""
    tok, diff, msk = _blank(B, T, 1)
    for b in range(B):
        p = 1
        while p + 3 <= T:
            k = int(rng.integers(k_min, k_max + 1))
            if p + k + 2 > T:
                k = T - p - 2
                if k < 1:
                    break
            g = rng.integers(0, n, size=k)
            s = 0
            for gi in g:
                s = mul[gi, s]
            tok[b, p:p + k] = BASE + g
            tok[b, p + k], tok[b, p + k + 1] = QUERY, BASE + n + s
            msk[b, p + k + 1], diff[b, p + k + 1] = True, k
            p += k + 2
    return tok, msk, diff


def make_mixed_tagged_batch(rng, B, n_ops, mul_a, n_a, mul_b, n_b, frac_a=0.5, force=None):
    """Each row is group A or group B (tagged format, disjoint token ranges).
    Layout: A ops BASE.., A states BASE+n_a.., B ops BASE+2n_a.., B states after.
    Returns (tok, tgt, msk, task [B]) with task 0 = A, 1 = B."""
    tok, tgt, msk = _blank(B, 1 + n_ops, 1)
    if force:
        is_b = np.full(B, force == "b")
    else:
        is_b = rng.random(B) >= frac_a
    for flag, mul, n, off in ((False, mul_a, n_a, BASE), (True, mul_b, n_b, BASE + 2 * n_a)):
        rows = np.where(is_b == flag)[0]
        if len(rows) == 0:
            continue
        g = rng.integers(0, n, size=(len(rows), n_ops))
        tok[rows, 1:] = off + g
        tgt[rows, 1:] = off + n + running_product(g, mul)
    msk[:, 1:] = True
    return tok, tgt, msk, is_b.astype(np.int64)


def make_keyed_group_batch(rng, B, mul, n, K, D, rho=0.0, K_max=None):
    """K registers, each a running product; D ops per register, interleaved; a
    fraction rho of the ops are cross-register ops s_k <- s_k * s_j; then every
    register is queried once.  Tokens: normal op [KEY_k, ELEM_g], cross op
    [KEY_k, XFROM, KEY_j], query [QUERY, KEY_k]; the target sits at the op's last
    token (the updated s_k) and at the query's key token (the final s_k).
    Vocab: KEY BASE.., ELEM BASE+K_max.., STATE BASE+K_max+n.. (K_max pins the
    layout across a K sweep).  One op schedule per call, shared by the rows.
    Returns (tok, tgt, msk, depth) with depth = ops that register has received."""
    K_max = K if K_max is None else K_max
    KEYB, ELEMB, STATEB = BASE, BASE + K_max, BASE + K_max + n
    n_ops = K * D
    order = np.repeat(np.arange(K), D)
    rng.shuffle(order)
    seen_before = [set(order[:t].tolist()) - {int(order[t])} for t in range(n_ops)]
    eligible = [t for t in range(n_ops) if seen_before[t]]
    cross = np.zeros(n_ops, dtype=bool)
    n_cross = int(round(rho * n_ops))
    if n_cross and eligible:
        cross[np.atleast_1d(rng.choice(eligible, size=min(n_cross, len(eligible)), replace=False))] = True
    src = [int(rng.choice(sorted(seen_before[t]))) if cross[t] else -1 for t in range(n_ops)]
    width = np.where(cross, 3, 2)
    start = 1 + np.concatenate(([0], np.cumsum(width)[:-1]))
    q0 = 1 + int(width.sum())
    tok, tgt, depth, msk = _blank(B, q0 + 2 * K, 2)
    g = rng.integers(0, n, size=(B, n_ops))
    state = np.zeros((B, K), dtype=np.int64)
    count = np.zeros(K, dtype=np.int64)
    for t in range(n_ops):
        k, p = int(order[t]), int(start[t])
        if cross[t]:
            state[:, k] = mul[state[:, k], state[:, src[t]]]
            tok[:, p], tok[:, p + 1], tok[:, p + 2] = KEYB + k, XFROM, KEYB + src[t]
        else:
            state[:, k] = mul[g[:, t], state[:, k]]
            tok[:, p], tok[:, p + 1] = KEYB + k, ELEMB + g[:, t]
        last = p + int(width[t]) - 1
        count[k] += 1
        tgt[:, last], msk[:, last], depth[:, last] = STATEB + state[:, k], True, count[k]
    for i, k in enumerate(rng.permutation(K)):
        p = q0 + 2 * i
        tok[:, p], tok[:, p + 1] = QUERY, KEYB + int(k)
        tgt[:, p + 1], msk[:, p + 1], depth[:, p + 1] = STATEB + state[:, int(k)], True, D
    return tok, tgt, msk, depth


# ============================================================================== k-hop / recall / parity
def make_khop_batch(rng, B, n_sym, n_q, k_max, sorted_pairs=False, ablate_pairs=False):
    """A planted Hamiltonian cycle given as shuffled [key ARROW succ] pairs, then
    queries [QUERY start k answer] with answer = succ^k(start).  k tokens sit at
    BASE.. (fixed across lengths), symbols follow.  Returns (tok, msk, diff [B, n_q])."""
    ktok, sym = BASE, BASE + k_max
    tok, msk = _blank(B, 1 + 3 * n_sym + 4 * n_q)
    diff = np.zeros((B, n_q), dtype=np.int64)
    for b in range(B):
        cyc = rng.permutation(n_sym)
        succ = np.empty(n_sym, dtype=np.int64)
        succ[cyc] = np.roll(cyc, -1)
        keys = cyc if sorted_pairs else rng.permutation(n_sym)
        body = np.stack((sym + keys, np.full(n_sym, ARROW), sym + succ[keys]), axis=1).reshape(-1)
        if ablate_pairs:
            body = rng.integers(sym, sym + n_sym, size=body.shape[0])
        tok[b, 1:1 + 3 * n_sym] = body
        p = 1 + 3 * n_sym
        for qi in range(n_q):
            a = start = int(rng.integers(0, n_sym))
            k = int(rng.integers(1, k_max + 1))
            for _ in range(k):
                a = succ[a]
            tok[b, p:p + 4] = (QUERY, sym + start, ktok + k - 1, sym + a)
            msk[b, p + 3], diff[b, qi] = True, k
            p += 4
    return tok, msk, diff


def make_niah_batch(rng, B, n_pairs, v_len, n_q, key_pool=512, val_pool=64, pairs_min=None):
    """[k ARROW v1..vL SEP] pairs, then queries [QUERY k v1..vL]: the model must
    emit the whole multi-token value.  Returns (tok, msk, diff) with diff = position
    inside the value (1..v_len)."""
    key0, val0 = BASE, BASE + key_pool
    T = 1 + n_pairs * (v_len + 3) + n_q * (v_len + 2)
    tok, diff, msk = _blank(B, T, 1)
    for b in range(B):
        npb = n_pairs if pairs_min is None else int(rng.integers(pairs_min, n_pairs + 1))
        keys = rng.choice(key_pool, size=npb, replace=False)
        vals = rng.integers(0, val_pool, size=(n_pairs, v_len))
        p = 1
        for i in rng.permutation(npb):
            tok[b, p], tok[b, p + 1] = key0 + keys[i], ARROW
            tok[b, p + 2:p + 2 + v_len] = val0 + vals[i]
            tok[b, p + 2 + v_len] = SEP
            p += v_len + 3
        for qi in rng.choice(npb, size=min(n_q, npb), replace=False):
            tok[b, p], tok[b, p + 1] = QUERY, key0 + keys[qi]
            tok[b, p + 2:p + 2 + v_len] = val0 + vals[qi]
            msk[b, p + 2:p + 2 + v_len] = True
            diff[b, p + 2:p + 2 + v_len] = np.arange(1, v_len + 1)
            p += v_len + 2
    return tok, msk, diff


def make_parity_batch(rng, B, n_ops):
    bits = rng.integers(0, 2, size=(B, n_ops))
    tok, msk = _blank(B, 1 + 2 * n_ops)
    tok[:, 1::2] = BASE + bits
    tok[:, 2::2] = BASE + 2 + np.bitwise_xor.accumulate(bits, axis=1)
    msk[:, 2::2] = True
    return tok, msk


# ============================================================================== cellular automata
CA_RULE = {90: np.array([0, 1, 0, 1, 1, 0, 1, 0], dtype=np.int64),
           110: np.array([0, 1, 1, 1, 0, 1, 1, 0], dtype=np.int64)}
CA_RULE_TOK = BASE + 2
CA_TIME_TOK = BASE + 4


def ca_rollout(rng, B, w, t, rule):
    """[B, t+1, w] space-time diagram from a random first row, periodic boundary."""
    table = CA_RULE[rule]
    rows = np.empty((B, t + 1, w), dtype=np.int64)
    rows[:, 0] = rng.integers(0, 2, size=(B, w))
    for k in range(t):
        cur = rows[:, k]
        rows[:, k + 1] = table[4 * np.roll(cur, 1, axis=1) + 2 * cur + np.roll(cur, -1, axis=1)]
    return rows


def ca_certify(rng, w, t, rule, B=4096):
    """(marginal of the answer bit at depth t, fraction of orbits whose row t already
    occurred earlier, i.e. deep queries that are secretly shallow)."""
    rows = ca_rollout(rng, B, w, t, rule)
    marg = float(rows[:, t].mean())
    if t == 0:
        return marg, 0.0
    repeat = (rows[:, :t] == rows[:, t][:, None, :]).all(-1).any(1)
    return marg, float(repeat.mean())


def ca_cell_ok(marg, short):
    return 0.4 <= marg <= 0.6 and short < 0.02


def make_ca_batch(rng, B, w, t, rule, fmt="silent", pad=0, gap=1):
    """silent: [BOS, RULE, TIME_t, row0, PAD x pad, QUERY x w] -> row_t at the QUERY
    slots.  trace: [BOS, RULE, row0..row_{t-1}] -> next row per cell.  leaky: the whole
    diagram with rows at multiples of `gap` (and rows 0, t) given, the rest to fill in."""
    rows = ca_rollout(rng, B, w, t, rule)
    rtok = CA_RULE_TOK + (0 if rule == 90 else 1)
    if fmt == "silent":
        tok, tgt, msk = _blank(B, 3 + 2 * w + pad, 1)
        tok[:, 1], tok[:, 2] = rtok, CA_TIME_TOK + t
        tok[:, 3:3 + w] = BASE + rows[:, 0]
        a = 3 + w + pad
        tok[:, a:], tgt[:, a:], msk[:, a:] = QUERY, BASE + rows[:, t], True
    elif fmt == "trace":
        tok, tgt, msk = _blank(B, 2 + t * w, 1)
        tok[:, 1] = rtok
        tok[:, 2:] = (BASE + rows[:, :t]).reshape(B, -1)
        tgt[:, 2:] = (BASE + rows[:, 1:]).reshape(B, -1)
        msk[:, 2:] = True
    elif fmt == "leaky":
        given = set(range(0, t + 1, max(1, gap))) | {0, t}
        tok, tgt, msk = _blank(B, 2 + (t + 1) * w, 1)
        tok[:, 1] = rtok
        for k in range(t + 1):
            c = slice(2 + k * w, 2 + (k + 1) * w)
            if k in given:
                tok[:, c] = BASE + rows[:, k]
            else:
                tok[:, c], tgt[:, c], msk[:, c] = QUERY, BASE + rows[:, k], True
    else:
        raise ValueError(f"ca fmt {fmt}")
    return tok, tgt, msk


# ============================================================================== match-3
def make_match3_batch(rng, B, n_ops, M=151, W=16, mask_from=None):
    """y_t = 1 iff some triple among the last W values (ending at x_t) sums to 0 mod M.
    Interleaved [BOS, x1, y1, ...]; only positions with a full window are scored."""
    x = rng.integers(0, M, size=(B, n_ops))
    y = np.zeros((B, n_ops), dtype=np.int64)
    for b in range(B):
        pair_count = np.zeros(M, dtype=np.int32)
        window = []
        for t in range(n_ops):
            v = int(x[b, t])
            if len(window) >= 2 and pair_count[(-v) % M] > 0:
                y[b, t] = 1
            for u in window:
                pair_count[(u + v) % M] += 1
            window.append(v)
            if len(window) > W - 1:
                old = window.pop(0)
                for u in window:
                    pair_count[(old + u) % M] -= 1
    tok, msk = _blank(B, 1 + 2 * n_ops)
    tok[:, 1::2], tok[:, 2::2] = BASE + x, BASE + M + y
    msk[:, 2::2] = True
    msk[:, :1 + 2 * (W if mask_from is None else mask_from)] = False
    return tok, msk


def match3_base_rate(M=151, W=16, n=200_000, seed=0):
    tok, msk = make_match3_batch(np.random.default_rng(seed), 8, n // 8, M=M, W=W)
    return float((tok[msk] - (BASE + M)).mean())


# ============================================================================== GF(p) linear algebra
MI_OPS = {"inv": 0, "solve": 1, "mul": 2}


def mi_op_tok(p, op):
    return BASE + p + MI_OPS[op]


def mi_size_tok(p, n):
    return BASE + p + 3 + n


def mi_vocab(p, n_max):
    return BASE + p + 3 + n_max + 1


def gf_inv_batch(A, p):
    """Batched Gauss-Jordan inverse over GF(p): A [B,n,n] -> (inverse, ok [B])."""
    B, n, _ = A.shape
    M = np.concatenate((A % p, np.broadcast_to(np.eye(n, dtype=np.int64), (B, n, n))), axis=2).copy()
    ok = np.ones(B, dtype=bool)
    rows = np.arange(B)
    for c in range(n):
        nonzero = M[:, c:, c] != 0
        ok &= nonzero.any(1)
        piv = c + nonzero.argmax(1)
        top, low = M[rows, c].copy(), M[rows, piv].copy()
        M[rows, c], M[rows, piv] = low, top
        lead = M[:, c, c] % p
        inv_lead = np.array([pow(int(v), p - 2, p) if v else 1 for v in lead], dtype=np.int64)
        M[:, c] = (M[:, c] * inv_lead[:, None]) % p
        factor = M[:, :, c].copy()
        factor[:, c] = 0
        M = (M - factor[:, :, None] * M[:, c][:, None, :]) % p
    return M[:, :, n:], ok


def gl_sample(rng, B, n, p):
    """B uniformly random invertible matrices over GF(p) with their inverses (rejection)."""
    A = rng.integers(0, p, size=(B, n, n))
    inv, ok = gf_inv_batch(A, p)
    for _ in range(200):
        bad = np.where(~ok)[0]
        if len(bad) == 0:
            return A, inv
        A[bad] = rng.integers(0, p, size=(len(bad), n, n))
        inv[bad], ok[bad] = gf_inv_batch(A[bad], p)
    raise RuntimeError("gl_sample: rejection stalled")


def make_matinv_batch(rng, B, n, p=2, op="inv", pad=0):
    """[BOS, OP, SIZE_n, A (row-major), extra, PAD x pad, QUERY x answer] -> answer at the
    QUERY slots.  inv: A^-1; solve: extra = b, answer x with Ax = b; mul: extra = B, answer AB."""
    A, Ainv = gl_sample(rng, B, n, p)
    nn = n * n
    if op == "inv":
        extra, ans = np.zeros((B, 0), dtype=np.int64), Ainv.reshape(B, nn)
    elif op == "solve":
        b = rng.integers(0, p, size=(B, n, 1))
        extra, ans = b.reshape(B, n), ((Ainv @ b) % p).reshape(B, n)
    elif op == "mul":
        Bm = rng.integers(0, p, size=(B, n, n))
        extra, ans = Bm.reshape(B, nn), ((A @ Bm) % p).reshape(B, nn)
    else:
        raise ValueError(op)
    ne, na = extra.shape[1], ans.shape[1]
    tok, tgt, msk = _blank(B, 3 + nn + ne + pad + na, 1)
    tok[:, 1], tok[:, 2] = mi_op_tok(p, op), mi_size_tok(p, n)
    tok[:, 3:3 + nn] = BASE + A.reshape(B, nn)
    tok[:, 3 + nn:3 + nn + ne] = BASE + extra
    a = 3 + nn + ne + pad
    tok[:, a:], tgt[:, a:], msk[:, a:] = QUERY, BASE + ans, True
    return tok, tgt, msk


def mi_certify(rng, n, p, op, B=2048):
    """(largest answer-symbol marginal, agreement of the answer with the trivial guess)."""
    tok, tgt, msk = make_matinv_batch(rng, B, n, p, op)
    ans = tgt[msk].reshape(B, -1) - BASE
    marg = max(float((ans == s).mean()) for s in range(p))
    nn = n * n
    guess = tok[:, 3:3 + nn] - BASE if op in ("inv", "mul") else tok[:, 3 + nn:3 + nn + n] - BASE
    return marg, float((ans == guess[:, :ans.shape[1]]).mean())


# ============================================================================== DFA state prediction
def dfa_lib(name):
    """(trans [n_states, n_sym], n_states, n_sym, in_crasp); trans[q, a] = next state."""
    if name in ("z2", "z3", "z5", "z10", "s3", "a5", "a4xz5"):
        mul, n = cayley(name)
        return np.asarray(mul).T.astype(np.int64), n, n, False
    table = {"flipflop": ([[0, 1], [0, 1]], False), "contains_a": ([[1, 0], [1, 1]], True),
             "contains_ab": ([[1, 0], [1, 2], [2, 2]], True),
             "count_a_ge3": ([[1, 0], [2, 1], [3, 2], [3, 3]], True)}
    if name not in table:
        raise ValueError(name)
    t, crasp = table[name]
    t = np.array(t, dtype=np.int64)
    return t, t.shape[0], t.shape[1], crasp


def make_dfa_batch(rng, B, T, trans, n_states, n_sym, sep=False):
    """sep=False: [BOS, a1..aT], target q_t at the symbol.  sep=True: [BOS, &, a1, &, ...]
    with the state predicted only at the separators (the one before a1 carries q0)."""
    a = rng.integers(0, n_sym, size=(B, T))
    q = np.empty((B, T), dtype=np.int64)
    prev = np.zeros(B, dtype=np.int64)
    for t in range(T):
        prev = trans[prev, a[:, t]]
        q[:, t] = prev
    if not sep:
        tok, tgt, msk = _blank(B, 1 + T, 1)
        tok[:, 1:], tgt[:, 1:], msk[:, 1:] = BASE + a, BASE + n_sym + q, True
        return tok, tgt, msk
    tok, tgt, msk = _blank(B, 2 + 2 * T, 1)
    tok[:, 1::2], tok[:, 2::2] = ARROW, BASE + a
    tgt[:, 1], tgt[:, 3::2] = BASE + n_sym, BASE + n_sym + q
    msk[:, 1::2] = True
    return tok, tgt, msk


# ============================================================================== circuit value problem
CVP_TOK_PER_GATE = 5
CVP_GATE = ["xormaj"]          # xormaj | copy | xor2 (depth-1 controls)


def cvp_vocab(n_max, m):
    return BASE + (m + n_max) + 2 + 2


def _gate(va, vb, vd, vc):
    kind = CVP_GATE[0]
    if kind == "copy":
        return va
    if kind == "xor2":
        return va ^ vc
    return vc ^ ((va + vb + vd) >= 2).astype(np.int64)


def make_cvp_batch(rng, B, n, m=32, fmt="tagged", pad=0, chain=1.0, n_queries=4, n_max=None,
                   n_topo=1, window=0, m_max=None, leak_every=0, addr="abs"):
    """Keyed circuit value problem over gates v_k = v_c XOR MAJ(v_a, v_b, v_d), in
    topological order.  Inputs [GID_k, BIT]; gates [GID_k, GID_a, GID_b, GID_d, GID_c].
    `chain` = probability that the carry operand c is gate k-1 (1.0: depth = gate index).
    tagged: the value is the target at each gate's last token, plus queries
    [QUERY, GID_k]; silent: no dense targets, PAD x pad, then queries.
    leak_every = g: after every g-th gate its value is appended as an input token.
    addr="rel": operands are written as how many gates back.  (m_max, n_max) pin the
    vocab layout over a curriculum.  n_topo > 1 splits the batch over independent
    circuits.  Returns (tok, tgt, msk, depth)."""
    if n_topo > 1:
        sizes = [B // n_topo + (i < B % n_topo) for i in range(n_topo)]
        parts = [_cvp_one(rng, s, n, m, fmt, pad, chain, n_queries, n_max, window, m_max, leak_every, addr)
                 for s in sizes if s > 0]
        return tuple(np.concatenate([p[i] for p in parts], axis=0) for i in range(4))
    return _cvp_one(rng, B, n, m, fmt, pad, chain, n_queries, n_max, window, m_max, leak_every, addr)


def _cvp_one(rng, B, n, m, fmt, pad, chain, n_queries, n_max, window, m_max, leak_every, addr):
    n_max = n if n_max is None else n_max
    m_max = m if m_max is None else m_max
    G = m + n
    gid = np.concatenate((np.arange(m), m_max + np.arange(n)))
    GIDB, BITB = BASE, BASE + m_max + n_max
    VALB = BITB + 2
    src = np.zeros((G, 4), dtype=np.int64)
    gate_depth = np.zeros(G, dtype=np.int64)
    for k in range(m, G):
        lo = max(0, k - window) if window else 0
        src[k, :3] = lo + rng.choice(k - lo, size=3, replace=(k - lo < 3))
        src[k, 3] = k - 1 if rng.random() < chain else int(rng.integers(lo, k))
        gate_depth[k] = 1 + gate_depth[src[k]].max()
    val = np.zeros((B, G), dtype=np.int64)
    val[:, :m] = rng.integers(0, 2, size=(B, m))
    for k in range(m, G):
        a, b, d, c = src[k]
        val[:, k] = _gate(val[:, a], val[:, b], val[:, d], val[:, c])
    q = min(n_queries, n)
    asked = np.array([G - 1]) if q <= 1 else np.concatenate(
        ([G - 1], rng.choice(np.arange(m, G - 1), size=q - 1, replace=False)))
    leaked = {k for k in range(m, G) if leak_every and fmt == "tagged" and (k - m + 1) % leak_every == 0}
    T = 1 + 2 * m + CVP_TOK_PER_GATE * n + len(leaked) + (pad if fmt == "silent" else 0) + 2 * q
    tok, tgt, depth, msk = _blank(B, T, 2)
    tok[:, 1:1 + 2 * m:2] = GIDB + gid[:m]
    tok[:, 2:2 + 2 * m:2] = BITB + val[:, :m]
    p = 1 + 2 * m
    for k in range(m, G):
        tok[:, p] = GIDB + gid[k]
        tok[:, p + 1:p + 5] = GIDB + ((k - src[k] - 1) if addr == "rel" else gid[src[k]])
        if fmt == "tagged":
            tgt[:, p + 4], msk[:, p + 4], depth[:, p + 4] = VALB + val[:, k], True, gate_depth[k]
        p += CVP_TOK_PER_GATE
        if k in leaked:
            tok[:, p] = BITB + val[:, k]
            p += 1
    if fmt == "silent":
        p += pad                                     # PAD tokens (already zero)
    for k in asked:
        k = int(k)
        tok[:, p], tok[:, p + 1] = QUERY, GIDB + ((G - 1 - k) if addr == "rel" else int(gid[k]))
        tgt[:, p + 1], msk[:, p + 1], depth[:, p + 1] = VALB + val[:, k], True, gate_depth[k]
        p += 2
    assert p == T
    return tok, tgt, msk, depth


def cvp_values_from_tokens(tok, m, n):
    """Re-evaluate a circuit from its tokens (default layout only).  -> (values, operands)."""
    G, GIDB, BITB = m + n, BASE, BASE + m + n
    vals = np.zeros((tok.shape[0], G), dtype=np.int64)
    vals[:, :m] = tok[:, 2:2 + 2 * m:2] - BITB
    p, ops = 1 + 2 * m, []
    for k in range(m, G):
        a, b, d, c = (tok[0, p + 1:p + 5] - GIDB).tolist()
        vals[:, k] = _gate(vals[:, a], vals[:, b], vals[:, d], vals[:, c])
        ops.append((a, b, d, c))
        p += CVP_TOK_PER_GATE
    return vals, ops


def cvp_certify(rng, n, m=32, chain=1.0, B=4096, n_batches=8, window=0):
    """Over the final gate: (max marginal, best agreement of copy / negate of one operand)."""
    marg = short = 0.0
    for _ in range(n_batches):
        tok, *_ = make_cvp_batch(rng, B, n, m=m, fmt="silent", pad=0, chain=chain, n_queries=1, window=window)
        vals, ops = cvp_values_from_tokens(tok, m, n)
        v = vals[:, -1]
        marg += max(v.mean(), 1 - v.mean())
        short += max(max((vals[:, x] == v).mean(), (vals[:, x] != v).mean()) for x in ops[-1])
    return marg / n_batches, short / n_batches


def cvp_cell_ok(marg, short):
    return marg < 0.65 and short < 0.75
