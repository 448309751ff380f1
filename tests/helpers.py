"""Shared builders of the seeded synthetic workloads used by the parity tests, the smoke check and the benchmark."""
import numpy as np


def chain_plus_branch(chain_rows, branch_rows):
    """Parent links of a tree with rows 0..chain_rows-1 a chain (row 0 the anchor) and branch_rows more rows forming a
    second chain that hangs off the anchor (the context-lookup branch)."""
    parent = [-1] + list(range(chain_rows - 1))
    for b in range(branch_rows):
        parent.append(0 if b == 0 else chain_rows + b - 1)
    return parent


def random_tree(rng, n, chain):
    """Rows 0..chain a chain, the rest attached to random earlier rows."""
    parent = [-1] + list(range(chain))
    for r in range(chain + 1, n):
        parent.append(int(rng.integers(0, r)))
    return parent[:n]


def layer_tensor_specs(lbm, cfg, full):
    """(tensor id, rows, cols, std, bias) of one layer, the order and the distributions of the synthetic weights."""
    H, I, D = cfg.hidden, cfg.intermediate, cfg.head_dim
    s = [(lbm.T_INPUT_NORM, 1, H, 0.02, 0.0), (lbm.T_POST_NORM, 1, H, 0.02, 0.0), (lbm.T_GATE, I, H, 0.02, 0.0),
         (lbm.T_UP, I, H, 0.02, 0.0), (lbm.T_DOWN, H, I, 0.02, 0.0)]
    if full:
        s += [(lbm.T_Q, cfg.heads * 2 * D, H, 0.02, 0.0), (lbm.T_K, cfg.kv_heads * D, H, 0.02, 0.0),
              (lbm.T_V, cfg.kv_heads * D, H, 0.02, 0.0), (lbm.T_O, H, cfg.heads * D, 0.02, 0.0),
              (lbm.T_Q_NORM, 1, D, 0.02, 0.0), (lbm.T_K_NORM, 1, D, 0.02, 0.0)]
    else:
        C, Vs, HV = cfg.conv_channels, cfg.value_size, cfg.lin_v_heads
        s += [(lbm.T_IN_QKV, C, H, 0.02, 0.0), (lbm.T_IN_Z, Vs, H, 0.02, 0.0), (lbm.T_OUT, H, Vs, 0.02, 0.0),
              (lbm.T_IN_A, HV, H, 0.02, 0.0), (lbm.T_IN_B, HV, H, 0.02, 0.0), (lbm.T_CONV, C, 4, 0.3, 0.0),
              (lbm.T_A_LOG, 1, HV, 0.5, 0.0), (lbm.T_DT_BIAS, 1, HV, 0.5, 0.0), (lbm.T_LIN_NORM, 1, cfg.lin_v_dim, 0.02, 1.0)]
    return s


def all_tensor_specs(lbm, cfg):
    out = [(-1, lbm.T_EMBED, cfg.vocab, cfg.hidden, 0.02, 0.0), (-1, lbm.T_FINAL_NORM, 1, cfg.hidden, 0.02, 0.0),
           (-1, lbm.T_LM_HEAD, cfg.vocab, cfg.hidden, 0.02, 0.0)]
    for l in range(cfg.layers):
        out += [(l,) + t for t in layer_tensor_specs(lbm, cfg, bool(cfg.full_attention[l]))]
    return out


def load_weights_from_host(lbm, lom, cfg, seed, targets):
    """Generates every tensor on the host with the oracle's generator and hands the same fp32 arrays to each target
    through set_tensor (the real loading path of both sides)."""
    for (layer, tensor, rows, cols, std, bias) in all_tensor_specs(lbm, cfg):
        a = lom.synth(seed, lom.weight_stream(layer, tensor), 0, rows * cols, std, bias, True).reshape(rows, cols)
        for t in targets:
            t.set_tensor(layer, tensor, a)


def map_pages(targets, slot, positions, page_tokens, first_page):
    """Maps consecutive pages first_page.. for `positions` positions of a slot on every target; returns pages used."""
    n = (positions + page_tokens - 1) // page_tokens
    idx = np.arange(n, dtype=np.int32)
    pages = np.arange(first_page, first_page + n, dtype=np.int32)
    for t in targets:
        t.kv_table_set(slot, idx, pages)
    return n


def toy_sequences(rng, vocab, contexts=(3, 37, 512, 1029), chain_rows=16, branch_rows=4):
    """The toy configuration's step: per sequence a 16-row chain plus a 4-row lookup branch off the anchor, token ids
    uniform over the vocabulary."""
    seqs = []
    for s, ctx in enumerate(contexts):
        parent = chain_plus_branch(chain_rows, branch_rows)
        tokens = rng.integers(0, vocab, size=len(parent)).astype(np.int32)
        seqs.append({"slot": s, "pos": int(ctx), "tokens": tokens, "parent": np.array(parent, np.int32),
                     "chain": chain_rows - 1})
    return seqs


def setup_sessions(targets, cfg, seqs, page_tokens, seed, extra_rows=32):
    """Page tables, synthetic KV for the context and synthetic DeltaNet state for every sequence, on every target."""
    page = 1
    for q in seqs:
        page += map_pages(targets, q["slot"], q["pos"] + extra_rows, page_tokens, page)
        for t in targets:
            if q["pos"] > 0:
                t.synth_kv(q["slot"], q["pos"], seed)
            t.synth_state(q["slot"], seed)
    return page
