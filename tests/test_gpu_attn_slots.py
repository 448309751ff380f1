"""The attention kernels' partial-result buffers hold one slot per (kv head, 512-key chunk) of a step's contexts and are sized
for the pool's positions.  Sessions that share pages (the prefix KV store) can hold more context between them than the pool
has pages for: such a step is refused on the host before anything is launched, and a context created with
options.attn_positions takes it."""
import ctypes as C

import numpy as np
import pytest


def shared_sessions(lb, attn_positions):
    cfg = lb.toy_config()
    ctx = lb.Context(cfg, sessions=4, max_context=40064, page_tokens=16, pool_pages=64, max_seqs=4, max_rows=128,
                     attn_positions=attn_positions)
    ctx.synth_weights(0)
    n_idx = 40064 // 16
    # every session maps its whole context onto the pool's 64 pages, over and over: far more context than the pool holds
    idx = np.arange(n_idx, dtype=np.int32)
    for slot in range(4):
        ctx.kv_table_set(slot, idx, (1 + (idx + slot) % 64).astype(np.int32))
        ctx.synth_state(slot, slot)
    ctx.synth_kv(0, 64 * 16, 0)  # fills the 64 pages through session 0's first 64 entries
    return cfg, ctx


def steps(pos, n_seq, vocab):
    rng = np.random.default_rng(pos)
    out = []
    for s in range(n_seq):
        tok = rng.integers(0, vocab, 6).astype(np.int32)
        out.append(dict(slot=s, pos=pos, tokens=tok, parent=np.arange(-1, 5, dtype=np.int32), chain=5))
    return out


@pytest.mark.gpu
def test_a_step_beyond_the_partial_buffers_is_refused_not_launched(gpu, lb):
    cfg, ctx = shared_sessions(lb, 0)
    L = lb.lib()
    cap = L.ling_b200_attn_slot_capacity(ctx.h)
    need = L.ling_b200_attn_slot_need(ctx.h, 40000)
    assert need == (40000 + 511) // 512 + 1 and 3 * need <= cap < 4 * need
    with pytest.raises(lb.LingError, match="attention partial slots"):
        ctx.verify_step(steps(40000, 4, cfg.vocab), lb.STEP_COMMIT)
    res = ctx.verify_step(steps(40000, 3, cfg.vocab), 0)  # three of them fit, and the context is as usable as before
    assert all(r.status == 0 for r in res)
    ctx.close()


@pytest.mark.gpu
def test_attn_positions_sizes_the_buffers_and_changes_no_result(gpu, lb):
    cfg, small = shared_sessions(lb, 0)
    a = small.verify_step(steps(40000, 3, cfg.vocab), 0)
    small.close()
    cfg, big = shared_sessions(lb, 4 * 40064)
    assert lb.lib().ling_b200_attn_slot_capacity(big.h) >= 4 * lb.lib().ling_b200_attn_slot_need(big.h, 40000)
    b = big.verify_step(steps(40000, 3, cfg.vocab), 0)
    for x, y in zip(a, b):
        assert x.status == 0 and y.status == 0 and x.n_path == y.n_path and list(x.out[:x.n_out]) == list(y.out[:y.n_out])
    res = big.verify_step(steps(40000, 4, cfg.vocab), 0)  # the step the small context refuses
    assert all(r.status == 0 for r in res)
    for x, y in zip(a, res[:3]):
        assert list(x.out[:x.n_out]) == list(y.out[:y.n_out])  # batch mates change nothing
    big.close()
