"""ctypes binding of the CPU oracle (libling_oracle.so) and of the reference's own host code (oracle/_ref).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline / reference
legs, as the checker.  The product (ling-engine_b200/) never imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libling_oracle.so")
REF = os.path.join(HERE, "_ref", "libling_ref.so")


REFCUDA = os.path.join(HERE, "_ref", "libling_refcuda.so")
REF_TREE_TESTS = os.path.join(HERE, "_ref", "ling-tree-tests")
REFQUANT = os.path.join(HERE, "_ref", "libling_refquant.so")


def build(ref=True, reference=None):
    """Compiles the oracle and, where a checkout of the reference project is named (`reference` or the environment's
    LING_REFERENCE), the reference's host sources and its sm_100a-buildable CUDA kernels behind C wrappers."""
    subprocess.run(["make", "-C", HERE, "-s"], check=True)
    reference = reference or os.environ.get("LING_REFERENCE", "")
    if ref and reference and os.path.isdir(reference):
        subprocess.run(["make", "-C", HERE, "-s", "ref", "ref_cuda", "ref_quant", "REF=" + reference], check=False)


_lo = None
_ref = None


def lo():
    global _lo
    if _lo is None:
        if not os.path.exists(LIB):
            build(ref=False)
        L = C.CDLL(LIB)
        L.lo_create.restype = C.c_void_p
        L.lo_e4m3_decode.restype = C.c_float
        L.lo_e4m3_encode.argtypes = [C.c_float]
        L.lo_e4m3_encode.restype = C.c_uint8
        L.lo_bf16_round.argtypes = [C.c_float]
        L.lo_bf16_round.restype = C.c_float
        L.lo_weight_stream.restype = C.c_uint64
        L.lo_synth.argtypes = [C.c_uint64, C.c_uint64, C.c_size_t, C.c_size_t, C.c_float, C.c_float, C.c_int,
                               C.POINTER(C.c_float)]
        _lo = L
    return _lo


def ref():
    """The reference's host code, or None where it was not built (e.g. on a machine without the reference project)."""
    global _ref
    if _ref is None and os.path.exists(REF):
        L = C.CDLL(REF)
        L.ref_kvpool_create.restype = C.c_void_p
        _ref = L
    return _ref


_refcuda = None


def refcuda():
    """The reference's own CUDA kernels (sm_100a build), or None where they were not built."""
    global _refcuda
    if _refcuda is None and os.path.exists(REFCUDA):
        L = C.CDLL(REFCUDA)
        L.refcuda_last_error.restype = C.c_char_p
        _refcuda = L
    return _refcuda


_refquant = None


def refquant():
    """The reference's host-side NVFP4 weight rounding (quantize_nvfp4), or None where it was not built.  The library
    carries unresolved references to parts of the reference that are not built here: it is opened with lazy binding."""
    global _refquant
    if _refquant is None and os.path.exists(REFQUANT):
        L = C.CDLL(REFQUANT, mode=os.RTLD_LAZY)
        L.refquant_last_error.restype = C.c_char_p
        _refquant = L
    return _refquant


def _ip(a):
    return a.ctypes.data_as(C.POINTER(C.c_int)) if a is not None else None


def _fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float)) if a is not None else None


def _bp(a):
    return a.ctypes.data_as(C.POINTER(C.c_ubyte)) if a is not None else None


def synth(seed, stream, offset, n, std, bias=0.0, bf16=True):
    out = np.zeros(n, np.float32)
    lo().lo_synth(seed, stream, offset, n, std, bias, 1 if bf16 else 0, _fp(out))
    return out


def weight_stream(layer, tensor):
    return lo().lo_weight_stream(layer, tensor)


def quant_rows(x, bf16_first=False):
    x = np.ascontiguousarray(x, np.float32)
    rows, cols = x.shape
    codes = np.zeros((rows, cols), np.uint8)
    scales = np.zeros((rows, (cols + 127) // 128), np.float32)
    lo().lo_quant_rows(_fp(x), rows, cols, 1 if bf16_first else 0, _bp(codes), _fp(scales))
    return codes, scales


def e4m3_decode_table():
    return np.array([lo().lo_e4m3_decode(C.c_uint8(c)) for c in range(256)], np.float32)


def gemm_fp8(x, w):
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    y = np.zeros((x.shape[0], w.shape[0]), np.float32)
    lo().lo_gemm_fp8(_fp(x), _fp(w), _fp(y), x.shape[0], w.shape[0], x.shape[1])
    return y


def argmax(logits):
    logits = np.ascontiguousarray(logits, np.float32)
    ids, vals = np.zeros(logits.shape[0], np.int32), np.zeros(logits.shape[0], np.float32)
    lo().lo_argmax(_fp(logits), logits.shape[0], logits.shape[1], _ip(ids), _fp(vals))
    return ids, vals


def gdn_prefill(Hk, HV, Dk, Dv, pre, convw, g, beta, state, conv):
    """conv over the rows + the delta rule token by token; returns post, core, and the advanced state and window."""
    pre, g, beta = (np.ascontiguousarray(a, np.float32) for a in (pre, g, beta))
    convw = np.ascontiguousarray(convw, np.float32)
    state, conv = np.array(state, np.float32, order="C"), np.array(conv, np.float32, order="C")
    M, C = pre.shape
    post, core = np.zeros((M, C), np.float32), np.zeros((M, HV * Dv), np.float32)
    lo().lo_gdn_prefill(Hk, HV, Dk, Dv, M, _fp(pre), _fp(convw), _fp(g), _fp(beta), _fp(state), _fp(conv), _fp(post), _fp(core))
    return post, core, state, conv


def topk_rows(x, k):
    x = np.ascontiguousarray(x, np.float32)
    ids, vals = np.zeros((x.shape[0], k), np.int32), np.zeros((x.shape[0], k), np.float32)
    lo().lo_topk_rows(_fp(x), x.shape[0], x.shape[1], k, _fp(vals), _ip(ids))
    return vals, ids


def bf16_round_np(a):
    """fp32 -> BF16 (round to nearest even) -> fp32."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32).view(np.float32)


def sparse_select(p, us, masks, dynamic, cap):
    """The sparse head's selection (src/core/sparse_head.cu:1-11,120-230; src/core/kernels.cuh:296-306): approx[n] = max over the
    rows m of bf16(p[m]) . bf16(us[n]) (float64 sums here), rows = every n a mask marks plus the `dynamic` best of the others (every
    tie at the threshold taken; if fewer unmarked rows than `dynamic` exist, none), ascending, at most cap.
    Returns (rows, approx, marked)."""
    pb = bf16_round_np(p).astype(np.float64)
    ub = bf16_round_np(us).astype(np.float64)
    approx = (ub @ pb.T).max(axis=1)
    marked = np.zeros(us.shape[0], bool)
    for m in np.atleast_2d(masks):
        marked |= np.asarray(m) != 0
    free = np.flatnonzero(~marked)
    take = marked.copy()
    if dynamic > 0 and len(free) >= dynamic:
        thr = np.sort(approx[free].astype(np.float32))[-dynamic]
        take[free[approx[free].astype(np.float32) >= thr]] = True
    return np.flatnonzero(take)[:cap].astype(np.int32), approx, marked


def selector_project(x, W):
    x, W = np.ascontiguousarray(x, np.float32), np.ascontiguousarray(W, np.float32)
    hp = np.zeros((x.shape[0], 256), np.float32)
    lo().lo_selector_project(_fp(x), _fp(W), x.shape[0], x.shape[1], _fp(hp))
    return hp


def selector_lattice(hp, cand, unary, P, S, anchor):
    hp, unary = np.ascontiguousarray(hp, np.float32), np.ascontiguousarray(unary, np.float32)
    cand = np.ascontiguousarray(cand, np.int32)
    P, S = np.ascontiguousarray(P, np.float32), np.ascontiguousarray(S, np.float32)
    scores = np.zeros((hp.shape[0], 16, 16), np.float32)
    lo().lo_selector_lattice(_fp(hp), _ip(cand), _fp(unary), _fp(P), _fp(S), int(anchor), hp.shape[0], _fp(scores))
    return scores


class Model:
    """The oracle's model + sessions; the same method names as the product binding's Context."""

    def __init__(self, cfg, opt, structs):
        self.cfg, self.opt, self.S = cfg, opt, structs
        self.h = C.c_void_p(lo().lo_create(C.byref(cfg), C.byref(opt)))
        self.last_rows = 0
        self.last_seqs = 0

    def close(self):
        if self.h:
            lo().lo_destroy(self.h)
            self.h = None

    def set_tensor(self, layer, tensor, a):
        a = np.ascontiguousarray(a, dtype=np.float32)
        rows, cols = (a.shape if a.ndim == 2 else (1, a.size))
        assert lo().lo_set_tensor(self.h, layer, tensor, _fp(a), rows, cols) == 0

    def synth_weights(self, seed):
        assert lo().lo_synth_weights(self.h, C.c_uint64(seed)) == 0

    def synth_weights_layers(self, seed, layers, head_rows):
        arr = np.ascontiguousarray(layers, np.int32)
        assert lo().lo_synth_weights_layers(self.h, C.c_uint64(seed), _ip(arr), len(arr), head_rows) == 0

    def get_matrix(self, layer, tensor, rows, cols):
        codes = np.zeros((rows, cols), np.uint8)
        scales = np.zeros((rows, (cols + 127) // 128), np.float32)
        assert lo().lo_get_matrix(self.h, layer, tensor, _bp(codes), _fp(scales), rows, cols) == 0
        return codes, scales

    def kv_table_set(self, slot, idx, pages):
        idx = np.ascontiguousarray(idx, np.int32)
        pages = np.ascontiguousarray(pages, np.int32)
        assert lo().lo_kv_table_set(self.h, slot, _ip(idx), _ip(pages), len(idx)) == 0

    def kv_write(self, slot, attn_layer, start, k, v):
        k = np.ascontiguousarray(k, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        assert lo().lo_kv_write(self.h, slot, attn_layer, start, k.shape[0], _fp(k), _fp(v)) == 0

    def kv_read(self, slot, attn_layer, start, n, codes=False):
        hk, d = self.cfg.kv_heads, self.cfg.head_dim
        if codes:
            kc, vc = np.zeros((n, hk, d), np.uint8), np.zeros((n, hk, d), np.uint8)
            ks, vs = np.zeros((n, hk), np.float32), np.zeros((n, hk), np.float32)
            lo().lo_kv_read(self.h, slot, attn_layer, start, n, None, None, _bp(kc), _fp(ks), _bp(vc), _fp(vs))
            return kc, ks, vc, vs
        k, v = np.zeros((n, hk, d), np.float32), np.zeros((n, hk, d), np.float32)
        lo().lo_kv_read(self.h, slot, attn_layer, start, n, _fp(k), _fp(v), None, None, None, None)
        return k, v

    def synth_kv(self, slot, n, seed):
        assert lo().lo_synth_kv(self.h, slot, n, C.c_uint64(seed)) == 0

    def state_write(self, slot, gdn_layer, state=None, conv=None):
        s = None if state is None else np.ascontiguousarray(state, np.float32)
        w = None if conv is None else np.ascontiguousarray(conv, np.float32)
        assert lo().lo_state_write(self.h, slot, gdn_layer, _fp(s), _fp(w)) == 0

    def state_read(self, slot, gdn_layer):
        c = self.cfg
        s = np.zeros((c.lin_v_heads, c.lin_k_dim, c.lin_v_dim), np.float32)
        w = np.zeros((c.conv_channels, 3), np.float32)
        assert lo().lo_state_read(self.h, slot, gdn_layer, _fp(s), _fp(w)) == 0
        return s, w

    def synth_state(self, slot, seed):
        assert lo().lo_synth_state(self.h, slot, C.c_uint64(seed)) == 0

    def state_hash(self, slot):
        h = C.c_uint64()
        lo().lo_state_hash(self.h, slot, C.byref(h))
        return h.value

    def verify_step(self, seqs, flags=1, make_steps=None):
        arr, keep = make_steps(seqs)
        res = (self.S.SeqResult * len(seqs))()
        assert lo().lo_verify_step(self.h, arr, len(seqs), flags, res) == 0
        self.last_rows = sum(len(s["tokens"]) for s in seqs)
        self.last_seqs = len(seqs)
        return list(res)

    def verify_step_sample(self, seqs, layers, head_rows, make_steps=None):
        arr, keep = make_steps(seqs)
        la = np.ascontiguousarray(layers, np.int32)
        assert lo().lo_verify_step_sample(self.h, arr, len(seqs), _ip(la), len(la), head_rows) == 0

    def attention(self, seqs, attn_layer, q, make_steps=None):
        arr, keep = make_steps(seqs)
        q = np.ascontiguousarray(q, np.float32)
        out = np.zeros_like(q)
        assert lo().lo_attention(self.h, arr, len(seqs), attn_layer, _fp(q), _fp(out)) == 0
        self.last_rows = sum(len(s["tokens"]) for s in seqs)
        self.last_seqs = len(seqs)
        return out

    def layer_forward(self, seqs, layer, h_in, head_rows=-1, make_steps=None):
        """One layer alone on the residual rows h_in (layer == cfg.layers: the final norm and the head)."""
        arr, keep = make_steps(seqs)
        h_in = np.ascontiguousarray(h_in, np.float32)
        out = np.zeros_like(h_in)
        assert lo().lo_layer_forward(self.h, arr, len(seqs), layer, _fp(h_in), _fp(out), head_rows) == 0
        self.last_rows = sum(len(s["tokens"]) for s in seqs)
        self.last_seqs = len(seqs)
        return out

    def mixer_forward(self, seqs, layer, h_in, make_steps=None):
        """The layer's mixer alone on the residual rows h_in (no feed-forward block)."""
        arr, keep = make_steps(seqs)
        h_in = np.ascontiguousarray(h_in, np.float32)
        out = np.zeros_like(h_in)
        assert lo().lo_mixer_forward(self.h, arr, len(seqs), layer, _fp(h_in), _fp(out)) == 0
        self.last_rows = sum(len(s["tokens"]) for s in seqs)
        self.last_seqs = len(seqs)
        return out

    def attn_prepare(self, seqs, attn_layer, qkv, make_steps=None):
        """attn_prepare alone: returns (q [rows][heads][D], k before the cache rounding [rows][kv_heads][D])."""
        arr, keep = make_steps(seqs)
        qkv = np.ascontiguousarray(qkv, np.float32)
        c = self.cfg
        q = np.zeros((qkv.shape[0], c.heads, c.head_dim), np.float32)
        k = np.zeros((qkv.shape[0], c.kv_heads, c.head_dim), np.float32)
        assert lo().lo_attn_prepare(self.h, arr, len(seqs), attn_layer, _fp(qkv), _fp(q), _fp(k)) == 0
        self.last_rows = sum(len(s["tokens"]) for s in seqs)
        self.last_seqs = len(seqs)
        return q, k

    def read_tree_desc(self, seq):
        t = self.S.TreeDesc()
        assert lo().lo_read_tree_desc(self.h, seq, C.byref(t)) == 0
        return t

    def read_packing(self):
        n, s = self.last_rows, self.last_seqs
        out = {"row0": np.zeros(s + 1, np.int32)}
        for k in ("token", "seq_of", "depth", "rope_pos", "cache_slot"):
            out[k] = np.zeros(n, np.int32)
        out["anc"] = np.zeros(n, np.uint32)
        lo().lo_read_packing(self.h, _ip(out["row0"]), _ip(out["token"]), _ip(out["seq_of"]), _ip(out["depth"]),
                             _ip(out["rope_pos"]), _ip(out["cache_slot"]), out["anc"].ctypes.data_as(C.POINTER(C.c_uint32)))
        return out

    def read_argmax(self):
        ids, vals = np.zeros(self.last_rows, np.int32), np.zeros(self.last_rows, np.float32)
        lo().lo_read_argmax(self.h, _ip(ids), _fp(vals))
        return ids, vals

    def read_logits(self):
        out = np.zeros((self.last_rows, self.cfg.vocab), np.float32)
        lo().lo_read_logits(self.h, _fp(out))
        return out

    def read_tap(self, layer):
        out = np.zeros((self.last_rows, self.cfg.hidden), np.float32)
        assert lo().lo_read_tap(self.h, layer, _fp(out)) == 0
        return out


# ---- NVFP4 (prefill chunk): values [rows][K/2] two a byte (low nibble first), E4M3 scales [rows][K/16]
def _vp(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def nvfp4_quantize_weight(w_bf16_bits, use_reference=False):
    """BF16 bit patterns [N][K] -> (values, scales, scale2) by the oracle, or by the reference's own quantize_nvfp4."""
    w = np.ascontiguousarray(w_bf16_bits, np.uint16)
    N, K = w.shape
    q, sf, s2 = np.zeros((N, K // 2), np.uint8), np.zeros((N, K // 16), np.uint8), C.c_float()
    if use_reference:
        rc = refquant().refquant_nvfp4(_vp(w), N, K, _bp(q), _bp(sf), C.byref(s2), None)
    else:
        rc = lo().lo_nvfp4_quantize_weight(_vp(w), N, K, _bp(q), _bp(sf), C.byref(s2))
    assert rc == 0
    return q, sf, s2.value


def nvfp4_quant_act(x, input_scale, up=None):
    x = np.ascontiguousarray(x, np.float32)
    up = None if up is None else np.ascontiguousarray(up, np.float32)
    M, K = x.shape
    q, sf = np.zeros((M, K // 2), np.uint8), np.zeros((M, K // 16), np.uint8)
    assert lo().lo_nvfp4_quant_act(_fp(x), _fp(up), M, K, C.c_float(input_scale), _bp(q), _bp(sf)) == 0
    return q, sf


def nvfp4_dequant(q, sf):
    q, sf = np.ascontiguousarray(q, np.uint8), np.ascontiguousarray(sf, np.uint8)
    rows, K = q.shape[0], q.shape[1] * 2
    out = np.zeros((rows, K), np.float32)
    lo().lo_nvfp4_dequant(_bp(q), _bp(sf), rows, K, _fp(out))
    return out


def nvfp4_gemm(xq, xs, wq, ws, alpha, y=None, ldy=None, accumulate=False):
    xq, xs, wq, ws = (np.ascontiguousarray(a, np.uint8) for a in (xq, xs, wq, ws))
    M, N, K = xq.shape[0], wq.shape[0], xq.shape[1] * 2
    ldy = ldy or N
    y = np.zeros((M, ldy), np.float32) if y is None else np.ascontiguousarray(y, np.float32).copy()
    assert lo().lo_nvfp4_gemm(_bp(xq), _bp(xs), M, _bp(wq), _bp(ws), N, K, C.c_float(alpha), _fp(y), ldy, 1 if accumulate else 0) == 0
    return y


def rmsnorm_rows(x, w_bf16_bits, eps):
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w_bf16_bits, np.uint16)
    out = np.zeros_like(x)
    lo().lo_rmsnorm_rows(_fp(x), _vp(w), x.shape[0], x.shape[1], C.c_float(eps), _fp(out))
    return out
