"""The oracle's own invariants on the toy configuration (no GPU).  They restate, on the CPU restatement, the exactness
properties the reference checks between execution modes (tools/ling_run.cpp:22-80 --spec-check/--batch-check and
tests/tree_tests.cu:64-188 in the reference project): a tree row is computed exactly as a chain holding its path would
compute it, a sequence's rows do not depend on its batch-mates, and a verify + commit of n accepted rows leaves the
state that n plain one-row steps leave."""
import numpy as np
import pytest

import helpers


@pytest.fixture(scope="module")
def toy(lb, lo):
    cfg = lb.toy_config()
    opt = lb.Options(4, 2048, 16, 512, 4, 128, 0, 0, 0, 128, 0)
    m = lo.Model(cfg, opt, lb)
    helpers.load_weights_from_host(lb, lo, cfg, 0, [m])
    return cfg, m


def fresh_sessions(m, cfg, seqs):
    helpers.setup_sessions([m], cfg, seqs, 16, 0)


def test_number_formats(lo):
    tab = lo.e4m3_decode_table()
    assert tab[0x7e] == 448.0 and tab[0x08] == 2.0 ** -6 and tab[0x01] == 2.0 ** -9 and np.isnan(tab[0x7f])
    enc = lo.lo().lo_e4m3_encode
    for c in range(256):
        if (c & 0x7f) != 0x7f:
            assert enc(float(tab[c])) == c
    assert enc(1e9) == 0x7e and enc(-1e9) == 0xfe and enc(464.0) == 0x7e      # saturating
    assert enc(2.0 ** -10) == 0 and enc(3 * 2.0 ** -10) == 2                   # ties to even in the subnormal range
    assert enc(1.0625) == 0x38 and enc(1.1875) == 0x3a                         # ties to even between 1, 1.125, 1.25
    x = np.array([[0.0] * 128 + [1.0, -3.0] + [0.5] * 126 + [7.0] * 10], np.float32)
    codes, scales = lo.quant_rows(x)
    assert scales.shape == (1, 3) and scales[0, 0] == 1.0 and scales[0, 1] == np.float32(3.0) / np.float32(448.0)
    assert (codes[0, :128] == 0).all() and tab[codes[0, 129]] * scales[0, 1] == -3.0
    assert (tab[codes[0, 256:]] * scales[0, 2] == 7.0).all()


def test_generator_is_counter_based(lo):
    a = lo.synth(3, 17, 0, 1000, 0.02)
    b = lo.synth(3, 17, 400, 100, 0.02)
    assert (a[400:500] == b).all() and abs(a.std() - 0.02) < 2e-3 and (lo.synth(4, 17, 0, 1000, 0.02) != a).any()
    z = lo.synth(0, 5, 0, 200000, 1.0, 0.0, False)
    assert abs(z.mean()) < 0.01 and abs(z.std() - 1.0) < 0.01


def test_tree_rows_equal_chain_rows(toy, lb):
    cfg, m = toy
    rng = np.random.default_rng(1)
    seqs = helpers.toy_sequences(rng, cfg.vocab, contexts=(37,))
    fresh_sessions(m, cfg, seqs)
    m.verify_step(seqs, flags=lb.STEP_KEEP_LOGITS, make_steps=lb.make_steps)
    tree_logits = m.read_logits()
    for rows in ([0] + list(range(16, 20)), list(range(16))):  # the lookup branch, then the chain, each as a plain chain
        q = dict(seqs[0], tokens=seqs[0]["tokens"][rows], parent=np.array([-1] + list(range(len(rows) - 1)), np.int32),
                 chain=len(rows) - 1)
        fresh_sessions(m, cfg, [q])
        m.verify_step([q], flags=lb.STEP_KEEP_LOGITS, make_steps=lb.make_steps)
        assert np.array_equal(m.read_logits(), tree_logits[rows])


def test_rows_do_not_depend_on_batch_mates(toy, lb):
    cfg, m = toy
    rng = np.random.default_rng(2)
    seqs = helpers.toy_sequences(rng, cfg.vocab)
    fresh_sessions(m, cfg, seqs)
    m.verify_step(seqs, flags=lb.STEP_KEEP_LOGITS, make_steps=lb.make_steps)
    batch = m.read_logits()
    row0 = m.read_packing()["row0"]
    for s in (1, 3):
        fresh_sessions(m, cfg, seqs)
        m.verify_step([seqs[s]], flags=lb.STEP_KEEP_LOGITS, make_steps=lb.make_steps)
        assert np.array_equal(m.read_logits(), batch[row0[s]:row0[s + 1]])


def test_verify_and_commit_equals_plain_steps(toy, lb):
    cfg, m = toy
    rng = np.random.default_rng(3)
    q = helpers.toy_sequences(rng, cfg.vocab, contexts=(37,))[0]
    path = [0, 16, 17]                                    # accept two rows of the lookup branch
    force = np.zeros(20, np.int32)
    force[0], force[16], force[17] = q["tokens"][16], q["tokens"][17], 4095
    fresh_sessions(m, cfg, [q])
    res = m.verify_step([dict(q, force=force)], flags=lb.STEP_COMMIT | lb.STEP_KEEP_LOGITS, make_steps=lb.make_steps)[0]
    assert list(res.path)[:res.n_path] == path and res.next_token == 4095
    assert list(res.out)[:res.n_out] == [int(q["tokens"][16]), int(q["tokens"][17]), 4095]
    logits = m.read_logits()
    state = [m.state_read(0, g) for g in range(3)]
    kv = m.kv_read(0, 0, 37, 3, codes=True)
    fresh_sessions(m, cfg, [q])
    for j, r in enumerate(path):                          # the same tokens, one plain one-row step each
        one = {"slot": 0, "pos": 37 + j, "tokens": q["tokens"][[r]], "parent": np.array([-1], np.int32), "chain": 0}
        m.verify_step([one], flags=lb.STEP_COMMIT | lb.STEP_KEEP_LOGITS, make_steps=lb.make_steps)
        assert np.array_equal(m.read_logits()[0], logits[r])
    for g in range(3):
        s, w = m.state_read(0, g)
        assert np.array_equal(s, state[g][0]) and np.array_equal(w, state[g][1])
    for a, b in zip(kv, m.kv_read(0, 0, 37, 3, codes=True)):
        assert np.array_equal(a, b)


def test_commit_leaves_other_sessions_and_rejected_state_alone(toy, lb):
    cfg, m = toy
    rng = np.random.default_rng(4)
    seqs = helpers.toy_sequences(rng, cfg.vocab)
    fresh_sessions(m, cfg, seqs)
    before = [m.state_hash(s) for s in range(4)]
    m.verify_step(seqs[:2], flags=0, make_steps=lb.make_steps)            # a verify without commit writes no state
    assert [m.state_hash(s) for s in range(4)] == before
    m.verify_step(seqs[:2], flags=lb.STEP_COMMIT, make_steps=lb.make_steps)
    after = [m.state_hash(s) for s in range(4)]
    assert after[0] != before[0] and after[1] != before[1] and after[2:] == before[2:]
