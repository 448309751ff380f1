"""ctypes binding of libling_b200.so, the C-ABI library of the B200 verify step.

The product is the shared library (CUDA C++ for sm_100a, see csrc/ and include/ling_b200.h); this module only loads it
for the Python-driven tests and benchmark.  There is no CPU path: if the library is missing, importing `lib()` raises.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libling_b200.so")

MAX_LAYERS, MAX_SEQS, MAX_TREE_ROWS, MAX_TREE_VARIANTS = 128, 64, 32, 32
TREE_LEAF, TREE_WRITE = 1 << 8, 1 << 9
STEP_COMMIT, STEP_KEEP_LOGITS, STEP_KEEP_TAPS = 1, 2, 4
OK, ERR_ARG, ERR_CUDA, ERR_POOL, ERR_DEVICE_FLAG, ERR_UNSUPPORTED = range(6)

(T_EMBED, T_FINAL_NORM, T_LM_HEAD, T_INPUT_NORM, T_POST_NORM, T_GATE, T_UP, T_DOWN, T_IN_QKV, T_IN_Z, T_OUT, T_IN_A,
 T_IN_B, T_CONV, T_A_LOG, T_DT_BIAS, T_LIN_NORM, T_Q, T_K, T_V, T_O, T_Q_NORM, T_K_NORM, T_COUNT) = range(24)
MATRIX_TENSORS = {T_LM_HEAD, T_GATE, T_UP, T_DOWN, T_IN_QKV, T_IN_Z, T_OUT, T_Q, T_K, T_V, T_O}


class ModelConfig(C.Structure):
    _fields_ = [("hidden", C.c_int), ("intermediate", C.c_int), ("layers", C.c_int), ("vocab", C.c_int),
                ("heads", C.c_int), ("kv_heads", C.c_int), ("head_dim", C.c_int), ("rotary_dim", C.c_int),
                ("rope_theta", C.c_float), ("eps", C.c_float),
                ("lin_k_heads", C.c_int), ("lin_v_heads", C.c_int), ("lin_k_dim", C.c_int), ("lin_v_dim", C.c_int),
                ("conv_kernel", C.c_int), ("full_attention", C.c_ubyte * MAX_LAYERS)]

    @property
    def conv_channels(self):
        return 2 * self.lin_k_heads * self.lin_k_dim + self.lin_v_heads * self.lin_v_dim

    @property
    def value_size(self):
        return self.lin_v_heads * self.lin_v_dim

    def attn_layers(self):
        return [l for l in range(self.layers) if self.full_attention[l]]

    def gdn_layers(self):
        return [l for l in range(self.layers) if not self.full_attention[l]]


class Options(C.Structure):
    _fields_ = [("sessions", C.c_int), ("max_context", C.c_int), ("page_tokens", C.c_int), ("pool_pages", C.c_int),
                ("max_seqs", C.c_int), ("max_rows", C.c_int), ("gemm_impl", C.c_int), ("use_graph", C.c_int),
                ("device", C.c_int), ("debug_rows", C.c_int), ("pdl", C.c_int), ("chain", C.c_int), ("gating_stream", C.c_int), ("attn_positions", C.c_int),
                ("fuse_swiglu", C.c_int), ("reserved", C.c_int * 1)]


class SeqStep(C.Structure):
    _fields_ = [("slot", C.c_int), ("pos", C.c_int), ("rope_delta", C.c_int), ("n_rows", C.c_int), ("chain", C.c_int),
                ("tokens", C.POINTER(C.c_int)), ("parent", C.POINTER(C.c_int)), ("force_argmax", C.POINTER(C.c_int))]


class SeqResult(C.Structure):
    _fields_ = [("status", C.c_int), ("n_path", C.c_int), ("path", C.c_int * MAX_TREE_ROWS), ("next_token", C.c_int),
                ("n_out", C.c_int), ("out", C.c_int * (MAX_TREE_ROWS + 1))]


class TreeDesc(C.Structure):
    _fields_ = [("n", C.c_int), ("depth", C.c_int * MAX_TREE_ROWS), ("var", C.c_int * MAX_TREE_ROWS), ("nvar", C.c_int),
                ("path", (C.c_int * MAX_TREE_ROWS) * MAX_TREE_VARIANTS), ("ngdn", C.c_int),
                ("gdn_len", C.c_int * MAX_TREE_VARIANTS), ("gdn_step", (C.c_int * (2 * MAX_TREE_ROWS)) * MAX_TREE_VARIANTS)]


class MemoryPlan(C.Structure):
    _fields_ = [("weights", C.c_size_t), ("per_session", C.c_size_t), ("sessions", C.c_size_t), ("scratch", C.c_size_t),
                ("kv_pool", C.c_size_t), ("session_count", C.c_int), ("kv_pool_pages", C.c_long), ("total", C.c_size_t),
                ("refused", C.c_int)]


def make_config(hidden, intermediate, layers, vocab, heads, kv_heads, head_dim, rotary_dim, lin_k_heads, lin_v_heads,
                lin_k_dim, lin_v_dim, full_attention, rope_theta=1e7, eps=1e-6):
    cfg = ModelConfig(hidden, intermediate, layers, vocab, heads, kv_heads, head_dim, rotary_dim, rope_theta, eps,
                      lin_k_heads, lin_v_heads, lin_k_dim, lin_v_dim, 4)
    for l, f in enumerate(full_attention):
        cfg.full_attention[l] = 1 if f else 0
    return cfg


def toy_config():
    """The CPU-runnable toy: 4 layers (0-2 gated DeltaNet, 3 gated GQA attention), hidden 256, 4 q / 1 kv heads of 64,
    DeltaNet 2 qk + 4 v heads of 64, FFN 704, vocabulary 4096."""
    return make_config(256, 704, 4, 4096, 4, 1, 64, 16, 2, 4, 64, 64, [0, 0, 0, 1])


def config_27b(layers=64):
    """The 27B-class hybrid: 3:1 gated DeltaNet (16 qk / 48 v heads, dim 128) to gated GQA attention (24 q / 4 kv heads,
    dim 256), hidden 5120, FFN 17408, vocabulary 248320."""
    return make_config(5120, 17408, layers, 248320, 24, 4, 256, 64, 16, 48, 128, 128,
                       [(l % 4) == 3 for l in range(layers)])


_lib = None


def lib():
    """Loads the library; raises (no fallback) when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError("libling_b200.so is missing: build it with `python ling-engine_b200/build.py` "
                           "(there is no CPU fallback)")
    L = C.CDLL(LIB_PATH)
    L.ling_b200_last_error.restype = C.c_char_p
    L.ling_b200_weight_bytes.restype = C.c_size_t
    L.ling_b200_weight_bytes.argtypes = [C.c_void_p]
    L.ling_b200_create.argtypes = [C.POINTER(ModelConfig), C.POINTER(Options), C.POINTER(C.c_void_p)]
    L.ling_b200_destroy.argtypes = [C.c_void_p]
    L.ling_b200_kvpool_create.restype = C.c_void_p
    for name in ("destroy", "capacity", "free_pages", "pending_pages", "refs", "needed", "ensure", "share", "truncate",
                 "unshare", "net_need", "resume_need", "reclaimable", "retain", "release", "retire"):
        getattr(L, "ling_b200_kvpool_" + name).argtypes = None
    _lib = L
    return L


def last_error():
    return lib().ling_b200_last_error().decode()


class LingError(RuntimeError):
    pass


def check(rc, what=""):
    if rc != OK:
        raise LingError("%s failed (status %d): %s" % (what, rc, last_error()))


def _ip(a):
    return a.ctypes.data_as(C.POINTER(C.c_int))


def _fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float)) if a is not None else None


def _bp(a):
    return a.ctypes.data_as(C.POINTER(C.c_ubyte)) if a is not None else None


def make_steps(seqs):
    """seqs: list of dicts {slot, pos, tokens, parent, chain, rope_delta=0, force=None} -> (ctypes array, keepalive)."""
    arr = (SeqStep * len(seqs))()
    keep = []
    for i, s in enumerate(seqs):
        tok = np.ascontiguousarray(s["tokens"], dtype=np.int32)
        par = np.ascontiguousarray(s["parent"], dtype=np.int32)
        keep += [tok, par]
        arr[i].slot, arr[i].pos, arr[i].rope_delta = s["slot"], s["pos"], s.get("rope_delta", 0)
        arr[i].n_rows, arr[i].chain = len(tok), s["chain"]
        arr[i].tokens, arr[i].parent = _ip(tok), _ip(par)
        if s.get("force") is not None:
            f = np.ascontiguousarray(s["force"], dtype=np.int32)
            keep.append(f)
            arr[i].force_argmax = _ip(f)
    return arr, keep


class Context:
    """One engine context on one GPU (ling_b200_create .. ling_b200_destroy)."""

    def __init__(self, cfg, sessions=4, max_context=2048, page_tokens=16, pool_pages=512, max_seqs=4, max_rows=128,
                 gemm_impl=None, use_graph=1, device=0, debug_rows=0, pdl=0, chain=0, gating_stream=0, attn_positions=0, fuse_swiglu=0):
        if gemm_impl is None:  # a debugging knob: LING_B200_GEMM_IMPL=1 runs the CUDA-core cross-check GEMM instead
            gemm_impl = int(os.environ.get("LING_B200_GEMM_IMPL", "0"))
        self.cfg = cfg
        self.opt = Options(sessions, max_context, page_tokens, pool_pages, max_seqs, max_rows, gemm_impl, use_graph,
                           device, debug_rows, pdl, chain)
        self.opt.gating_stream = gating_stream
        self.opt.attn_positions = attn_positions
        self.opt.fuse_swiglu = fuse_swiglu
        self.h = C.c_void_p()
        rc = lib().ling_b200_create(C.byref(cfg), C.byref(self.opt), C.byref(self.h))
        if rc != OK:
            err = last_error()
            if self.h:
                lib().ling_b200_destroy(self.h)
            self.h = None
            raise LingError("ling_b200_create failed (status %d): %s" % (rc, err))
        self.last_rows = 0
        self.last_seqs = 0

    def sibling(self, max_seqs, max_rows):
        """A second set of step buffers on this context's weights, KV pool and sessions (ling_b200_create_sibling): for work that
        runs beside this context's verify steps.  Close it before this context."""
        sib = Context.__new__(Context)
        sib.cfg, sib.opt, sib.h, sib.last_rows, sib.last_seqs, sib.parent = self.cfg, self.opt, C.c_void_p(), 0, 0, self
        L = lib()
        L.ling_b200_create_sibling.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]
        rc = L.ling_b200_create_sibling(self.h, max_seqs, max_rows, C.byref(sib.h))
        if rc != OK:
            err = last_error()
            if sib.h:
                L.ling_b200_destroy(sib.h)
            sib.h = None
            raise LingError("ling_b200_create_sibling failed (status %d): %s" % (rc, err))
        return sib

    def close(self):
        if self.h:
            lib().ling_b200_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- weights
    def set_tensor(self, layer, tensor, a):
        a = np.ascontiguousarray(a, dtype=np.float32)
        rows, cols = (a.shape if a.ndim == 2 else (1, a.size))
        check(lib().ling_b200_set_tensor(self.h, layer, tensor, _fp(a), rows, cols), "set_tensor")

    def synth_weights(self, seed):
        check(lib().ling_b200_synth_weights(self.h, C.c_uint64(seed)), "synth_weights")

    def get_matrix(self, layer, tensor, rows, cols):
        codes = np.zeros((rows, cols), np.uint8)
        scales = np.zeros((rows, (cols + 127) // 128), np.float32)
        check(lib().ling_b200_get_matrix(self.h, layer, tensor, _bp(codes), _fp(scales), rows, cols), "get_matrix")
        return codes, scales

    def weight_bytes(self):
        return lib().ling_b200_weight_bytes(self.h)

    # ---- sessions
    def kv_table_set(self, slot, idx, pages):
        idx = np.ascontiguousarray(idx, np.int32)
        pages = np.ascontiguousarray(pages, np.int32)
        check(lib().ling_b200_kv_table_set(self.h, slot, _ip(idx), _ip(pages), len(idx)), "kv_table_set")

    def kv_pages_copy(self, src, dst):
        src = np.ascontiguousarray(src, np.int32)
        dst = np.ascontiguousarray(dst, np.int32)
        check(lib().ling_b200_kv_pages_copy(self.h, _ip(src), _ip(dst), len(src)), "kv_pages_copy")

    def kv_write(self, slot, attn_layer, start, k, v):
        k = np.ascontiguousarray(k, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        check(lib().ling_b200_kv_write(self.h, slot, attn_layer, start, k.shape[0], _fp(k), _fp(v)), "kv_write")

    def kv_read(self, slot, attn_layer, start, n, codes=False):
        hk, d = self.cfg.kv_heads, self.cfg.head_dim
        if codes:
            kc, vc = np.zeros((n, hk, d), np.uint8), np.zeros((n, hk, d), np.uint8)
            ks, vs = np.zeros((n, hk), np.float32), np.zeros((n, hk), np.float32)
            check(lib().ling_b200_kv_read(self.h, slot, attn_layer, start, n, None, None, _bp(kc), _fp(ks), _bp(vc), _fp(vs)),
                  "kv_read")
            return kc, ks, vc, vs
        k, v = np.zeros((n, hk, d), np.float32), np.zeros((n, hk, d), np.float32)
        check(lib().ling_b200_kv_read(self.h, slot, attn_layer, start, n, _fp(k), _fp(v), None, None, None, None), "kv_read")
        return k, v

    def synth_kv(self, slot, n, seed):
        check(lib().ling_b200_synth_kv(self.h, slot, n, C.c_uint64(seed)), "synth_kv")

    def state_write(self, slot, gdn_layer, state=None, conv=None):
        s = None if state is None else np.ascontiguousarray(state, np.float32)
        w = None if conv is None else np.ascontiguousarray(conv, np.float32)
        check(lib().ling_b200_state_write(self.h, slot, gdn_layer, _fp(s), _fp(w)), "state_write")

    def state_read(self, slot, gdn_layer):
        c = self.cfg
        s = np.zeros((c.lin_v_heads, c.lin_k_dim, c.lin_v_dim), np.float32)
        w = np.zeros((c.conv_channels, 3), np.float32)
        check(lib().ling_b200_state_read(self.h, slot, gdn_layer, _fp(s), _fp(w)), "state_read")
        return s, w

    def synth_state(self, slot, seed):
        check(lib().ling_b200_synth_state(self.h, slot, C.c_uint64(seed)), "synth_state")

    def state_hash(self, slot):
        h = C.c_uint64()
        check(lib().ling_b200_state_hash(self.h, slot, C.byref(h)), "state_hash")
        return h.value

    # ---- the step
    def verify_step(self, seqs, flags=STEP_COMMIT):
        arr, keep = make_steps(seqs)
        res = (SeqResult * len(seqs))()
        check(lib().ling_b200_verify_step(self.h, arr, len(seqs), flags, res), "verify_step")
        self.last_rows = sum(len(s["tokens"]) for s in seqs)
        self.last_seqs = len(seqs)
        return list(res)

    def stage(self, seqs, flags=STEP_COMMIT):
        arr, keep = make_steps(seqs)
        check(lib().ling_b200_step_stage(self.h, arr, len(seqs), flags), "step_stage")
        self.last_rows = sum(len(s["tokens"]) for s in seqs)
        self.last_seqs = len(seqs)

    def launch(self):
        check(lib().ling_b200_step_launch(self.h), "step_launch")

    def fetch(self):
        res = (SeqResult * self.last_seqs)()
        check(lib().ling_b200_step_fetch(self.h, res), "step_fetch")
        return list(res)

    def attention(self, seqs, attn_layer, q):
        """One attention layer alone on the slot's cache: q [rows][heads][head_dim] -> out, before the output gate."""
        arr, keep = make_steps(seqs)
        q = np.ascontiguousarray(q, np.float32)
        out = np.zeros_like(q)
        check(lib().ling_b200_attention_host(self.h, arr, len(seqs), attn_layer, _fp(q), _fp(out)), "attention_host")
        self.last_rows = sum(len(s["tokens"]) for s in seqs)
        self.last_seqs = len(seqs)
        return out

    def attn_prepare(self, seqs, attn_layer, qkv):
        """attn_prepare alone: qkv [rows][heads*2*D + 2*kv_heads*D] -> q [rows][heads][D]; K and V go to the cache."""
        arr, keep = make_steps(seqs)
        qkv = np.ascontiguousarray(qkv, np.float32)
        q = np.zeros((qkv.shape[0], self.cfg.heads, self.cfg.head_dim), np.float32)
        check(lib().ling_b200_attn_prepare_host(self.h, arr, len(seqs), attn_layer, _fp(qkv), _fp(q)), "attn_prepare_host")
        self.last_rows = sum(len(s["tokens"]) for s in seqs)
        self.last_seqs = len(seqs)
        return q

    def prefill_attention(self, slot, attn_layer, pos0, qkv):
        """Attention over a prefill chunk's rows at positions pos0.. of one session, in 32-row slices through the step's kernels:
        qkv [M][heads*2*D + 2*kv_heads*D] -> gated output [M][heads][D]; the rows' K and V go to the cache."""
        qkv = np.ascontiguousarray(qkv, np.float32)
        out = np.zeros((qkv.shape[0], self.cfg.heads, self.cfg.head_dim), np.float32)
        check(lib().ling_b200_prefill_attention_host(self.h, slot, attn_layer, pos0, qkv.shape[0], _fp(qkv), _fp(out)), "prefill_attention_host")
        return out

    def chunk_attention_layer(self, slot, layer, pos0, h):
        """A full-attention layer's whole mixer over a prefill chunk's residual rows h [M][hidden] at positions pos0.. of one
        session (norm, FP8 q|k|v, prepare, attention in 32-row chains, gate, FP8 o, residual add): returns the rows after it."""
        h = np.array(h, np.float32, order="C")
        check(lib().ling_b200_chunk_attention_layer_host(self.h, slot, layer, pos0, h.shape[0], _fp(h)), "chunk_attention_layer_host")
        return h

    def chunk_attention_layer_profile(self, slot, layer, pos0, M):
        """Device milliseconds of one chunk attention layer by kernel family, and the number of chain launches."""
        ms, passes = (C.c_float * 8)(), C.c_int(0)
        check(lib().ling_b200_chunk_attention_layer_profile(self.h, slot, layer, pos0, M, ms, C.byref(passes)), "chunk_attention_layer_profile")
        return {"projections": ms[0], "attention": ms[1], "combine": ms[2], "norms": ms[3], "prepare": ms[5]}, passes.value

    def read_tree_desc(self, seq):
        t = TreeDesc()
        check(lib().ling_b200_read_tree_desc(self.h, seq, C.byref(t)), "read_tree_desc")
        return t

    def read_packing(self):
        n, s = self.last_rows, self.last_seqs
        out = {"row0": np.zeros(s + 1, np.int32)}
        for k in ("token", "seq_of", "depth", "rope_pos", "cache_slot"):
            out[k] = np.zeros(n, np.int32)
        out["anc"] = np.zeros(n, np.uint32)
        check(lib().ling_b200_read_packing(self.h, _ip(out["row0"]), _ip(out["token"]), _ip(out["seq_of"]), _ip(out["depth"]),
                                           _ip(out["rope_pos"]), _ip(out["cache_slot"]),
                                           out["anc"].ctypes.data_as(C.POINTER(C.c_uint32))), "read_packing")
        return out

    def read_argmax(self):
        ids, vals = np.zeros(self.last_rows, np.int32), np.zeros(self.last_rows, np.float32)
        check(lib().ling_b200_read_argmax(self.h, _ip(ids), _fp(vals)), "read_argmax")
        return ids, vals

    def read_logits(self):
        out = np.zeros((self.last_rows, self.cfg.vocab), np.float32)
        check(lib().ling_b200_read_logits(self.h, _fp(out)), "read_logits")
        return out

    def read_tap(self, layer):
        out = np.zeros((self.last_rows, self.cfg.hidden), np.float32)
        check(lib().ling_b200_read_tap(self.h, layer, _fp(out)), "read_tap")
        return out

    # ---- timing
    def timer_begin(self):
        check(lib().ling_b200_timer_begin(self.h), "timer_begin")

    def timer_end(self):
        ms = C.c_float()
        check(lib().ling_b200_timer_end(self.h, C.byref(ms)), "timer_end")
        return ms.value

    def gemm_chain_ms(self, iters=5):
        ms = C.c_float()
        check(lib().ling_b200_gemm_chain_ms(self.h, iters, C.byref(ms)), "gemm_chain_ms")
        return ms.value

    def profile_step(self):
        ms = (C.c_float * 8)()
        n = C.c_int()
        check(lib().ling_b200_profile_step(self.h, ms, C.byref(n)), "profile_step")
        return list(ms), n.value

    def launch_count(self):
        return lib().ling_b200_step_launch_count(self.h)

    def flush_l2(self):
        check(lib().ling_b200_flush_l2(self.h), "flush_l2")

    def sync(self):
        check(lib().ling_b200_sync(self.h), "sync")


# ---- kernel-level helpers (host buffers in, host buffers out)
def gemm_fp8(x, w, impl=0, splits=0, device=0):
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    y = np.zeros((x.shape[0], w.shape[0]), np.float32)
    check(lib().ling_b200_gemm_fp8_host(device, impl, splits, _fp(x), _fp(w), _fp(y), x.shape[0], w.shape[0], x.shape[1]),
          "gemm_fp8_host")
    return y


def gemm_fp8_bench(M, N, K, impl=0, splits=0, iters=20, device=0):
    ms = C.c_float()
    check(lib().ling_b200_gemm_fp8_bench(device, impl, splits, M, N, K, iters, C.byref(ms)), "gemm_fp8_bench")
    return ms.value


def gdn_fused(Hk, HV, Dk, Dv, trees, inp, convw, g, beta, state, conv, norm_w, eps=1e-6, device=0):
    """The step's single DeltaNet kernel on host buffers.  trees: list of (parent list, chain) per sequence; inp
    [rows][C + HV*Dv]; state [n_seqs][HV][Dk][Dv]; conv [n_seqs][C][3].  Returns pre, post, core, codes, scales."""
    n_rows = np.array([len(p) for p, _ in trees], np.int32)
    chain = np.array([c for _, c in trees], np.int32)
    parent = np.concatenate([np.asarray(p, np.int32) for p, _ in trees]).astype(np.int32)
    rows, Cn, Vs = int(n_rows.sum()), 2 * Hk * Dk + HV * Dv, HV * Dv
    arrs = [np.ascontiguousarray(a, np.float32) for a in (inp, convw, g, beta, state, conv, norm_w)]
    pre, post = np.zeros((rows, Cn), np.float32), np.zeros((rows, Cn), np.float32)
    core = np.zeros((rows, Vs), np.float32)
    codes, scales = np.zeros((rows, Vs), np.uint8), np.zeros((rows, Vs // 128), np.float32)
    check(lib().ling_b200_gdn_fused_host(device, Hk, HV, Dk, Dv, len(trees), _ip(n_rows), _ip(chain), _ip(parent),
                                         *[_fp(a) for a in arrs], C.c_float(eps), _fp(pre), _fp(post), _fp(core), _bp(codes),
                                         _fp(scales)), "gdn_fused_host")
    return pre, post, core, codes, scales


# ---- NVFP4 operands of the prefill chunk (values [rows][K/2] two a byte, E4M3 scales [rows][K/16], fp32 tensor scale)
def to_bf16_bits(x):
    """fp32 array -> BF16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def _up(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def quantize_nvfp4(w_bf16_bits, device=0):
    w = np.ascontiguousarray(w_bf16_bits, np.uint16)
    N, K = w.shape
    q, sf, s2 = np.zeros((N, K // 2), np.uint8), np.zeros((N, K // 16), np.uint8), C.c_float()
    check(lib().ling_b200_quantize_nvfp4_host(device, _up(w), N, K, _bp(q), _bp(sf), C.byref(s2)), "quantize_nvfp4_host")
    return q, sf, s2.value


def quant_act_nvfp4(x, input_scale, up=None, device=0):
    x = np.ascontiguousarray(x, np.float32)
    up = None if up is None else np.ascontiguousarray(up, np.float32)
    M, K = x.shape
    q, sf = np.zeros((M, K // 2), np.uint8), np.zeros((M, K // 16), np.uint8)
    check(lib().ling_b200_quant_act_nvfp4_host(device, _fp(x), _fp(up), M, K, C.c_float(input_scale), _bp(q), _bp(sf)),
          "quant_act_nvfp4_host")
    return q, sf


def rmsnorm_quant_nvfp4(x, w_bf16_bits, eps, input_scale, want_out=True, device=0):
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w_bf16_bits, np.uint16)
    M, H = x.shape
    out = np.zeros((M, H), np.float32) if want_out else None
    q, sf = np.zeros((M, H // 2), np.uint8), np.zeros((M, H // 16), np.uint8)
    check(lib().ling_b200_rmsnorm_quant_nvfp4_host(device, _fp(x), _up(w), _fp(out), M, H, C.c_float(eps), C.c_float(input_scale),
                                                   _bp(q), _bp(sf)), "rmsnorm_quant_nvfp4_host")
    return out, q, sf


def prefill_gemm_nvfp4(xq, xs, wq, ws, alpha, y=None, ldy=None, accumulate=False, device=0):
    """y [M][ldy] (columns [0, N) written).  y given: used as the starting contents (and added to with accumulate)."""
    xq, xs, wq, ws = (np.ascontiguousarray(a, np.uint8) for a in (xq, xs, wq, ws))
    M, N, K = xq.shape[0], wq.shape[0], xq.shape[1] * 2
    ldy = ldy or N
    y = np.zeros((M, ldy), np.float32) if y is None else np.ascontiguousarray(y, np.float32).copy()
    check(lib().ling_b200_prefill_gemm_nvfp4_host(device, _bp(xq), _bp(xs), M, _bp(wq), _bp(ws), C.c_float(alpha), _fp(y), ldy, N, K,
                                                  1 if accumulate else 0), "prefill_gemm_nvfp4_host")
    return y


def prefill_swiglu_nvfp4(xq, xs, gq, gs, alpha_gate, uq, us, alpha_up, out_input_scale, device=0):
    xq, xs, gq, gs, uq, us = (np.ascontiguousarray(a, np.uint8) for a in (xq, xs, gq, gs, uq, us))
    M, N, K = xq.shape[0], gq.shape[0], xq.shape[1] * 2
    q, sf = np.zeros((M, N // 2), np.uint8), np.zeros((M, N // 16), np.uint8)
    check(lib().ling_b200_prefill_swiglu_nvfp4_host(device, _bp(xq), _bp(xs), M, _bp(gq), _bp(gs), C.c_float(alpha_gate), _bp(uq),
                                                    _bp(us), C.c_float(alpha_up), N, K, C.c_float(out_input_scale), _bp(q), _bp(sf)),
          "prefill_swiglu_nvfp4_host")
    return q, sf


def nvfp4_pair_mode(mode):
    """0: one CTA per tile; 1: the two-CTA (cta_group::2) form.  Returns the previous setting."""
    return lib().ling_b200_nvfp4_pair_mode(int(mode))


def nvfp4_gemm_bench(M, N, K, fused=False, iters=10, device=0, shares=False):
    """ms per launch; with shares, also the kernel's own cycle shares (issuer waiting for stages, issuer waiting for the
    epilogue, one epilogue warp busy) of a CTA's time."""
    ms, sh = C.c_float(), (C.c_double * 3)()
    check(lib().ling_b200_nvfp4_gemm_bench(device, M, N, K, 1 if fused else 0, iters, C.byref(ms), sh if shares else None),
          "nvfp4_gemm_bench")
    return (ms.value, list(sh)) if shares else ms.value


def fp4_tensor_peak(iters=20000, device=0, mode=0):
    tf, ms = C.c_float(), C.c_float()
    check(lib().ling_b200_fp4_tensor_peak(device, iters, mode, C.byref(tf), C.byref(ms)), "fp4_tensor_peak")
    return tf.value, ms.value


class Nvfp4Ffn:
    """The prefill chunk's NVFP4 feed-forward stack on the device (synthetic weights), on a stream of its own."""

    def __init__(self, layers, hidden, intermediate, max_rows, seed=0, device=0):
        self.h = C.c_void_p()
        self.layers, self.hidden, self.intermediate, self.max_rows = layers, hidden, intermediate, max_rows
        L = lib()
        L.ling_b200_nvfp4_ffn_create.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint64, C.POINTER(C.c_void_p)]
        for n in ("destroy", "set_residual", "launch", "set_ctas", "wait", "forward", "read_layer"):
            getattr(L, "ling_b200_nvfp4_ffn_" + n).argtypes = None
        check(L.ling_b200_nvfp4_ffn_create(device, layers, hidden, intermediate, max_rows, seed, C.byref(self.h)), "nvfp4_ffn_create")

    def close(self):
        if self.h:
            lib().ling_b200_nvfp4_ffn_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_residual(self, h):
        h = np.ascontiguousarray(h, np.float32)
        check(lib().ling_b200_nvfp4_ffn_set_residual(self.h, _fp(h), h.shape[0]), "nvfp4_ffn_set_residual")

    def add_mixers(self, k_heads, v_heads, full_every=4, seed=0):
        """The DeltaNet layers' prefill-path mixers in front of their feed-forward blocks (every layer but each full_every-th)."""
        check(lib().ling_b200_nvfp4_ffn_add_mixers(self.h, k_heads, v_heads, full_every, C.c_uint64(seed)), "nvfp4_ffn_add_mixers")

    def attach_context(self, ctx, slot, pos0, full_every=4):
        """The full-attention layers' mixers (each full_every-th layer) through a verify context's own projections and attention
        kernels: the chunk is positions pos0.. of the context's session `slot`."""
        check(lib().ling_b200_nvfp4_ffn_attach_context(self.h, ctx.h, slot, pos0, full_every), "nvfp4_ffn_attach_context")
        self._ctx = ctx  # keeps the context alive as long as the stack

    def launch(self, rows, repeats=1):
        check(lib().ling_b200_nvfp4_ffn_launch(self.h, rows, repeats), "nvfp4_ffn_launch")

    def set_ctas(self, ctas):
        check(lib().ling_b200_nvfp4_ffn_set_ctas(self.h, ctas), "nvfp4_ffn_set_ctas")

    def wait(self):
        ms = C.c_float()
        check(lib().ling_b200_nvfp4_ffn_wait(self.h, C.byref(ms)), "nvfp4_ffn_wait")
        return ms.value

    def forward(self, h):
        h = np.ascontiguousarray(h, np.float32)
        out = np.zeros_like(h)
        check(lib().ling_b200_nvfp4_ffn_forward(self.h, _fp(h), h.shape[0], _fp(out)), "nvfp4_ffn_forward")
        return out

    def read_layer(self, layer):
        H, I = self.hidden, self.intermediate
        norm = np.zeros(H, np.uint16)
        gq, gs = np.zeros((I, H // 2), np.uint8), np.zeros((I, H // 16), np.uint8)
        uq, us = np.zeros((I, H // 2), np.uint8), np.zeros((I, H // 16), np.uint8)
        dq, ds = np.zeros((H, I // 2), np.uint8), np.zeros((H, I // 16), np.uint8)
        sc = np.zeros(5, np.float32)
        check(lib().ling_b200_nvfp4_ffn_read_layer(self.h, layer, _up(norm), _bp(gq), _bp(gs), _bp(uq), _bp(us), _bp(dq), _bp(ds),
                                                   _fp(sc)), "nvfp4_ffn_read_layer")
        return dict(norm=norm, gate=(gq, gs), up=(uq, us), down=(dq, ds), in_scale=float(sc[0]), mid_scale=float(sc[1]),
                    s_gate=float(sc[2]), s_up=float(sc[3]), s_down=float(sc[4]))


def gdn_prefill(Hk, HV, Dk, Dv, pre, convw_bits, g, beta, state, conv, device=0):
    """The prefill path's DeltaNet core over the rows of one sequence (ling_b200_gdn_prefill_host): returns post, core and the
    advanced state and window."""
    pre, g, beta = (np.ascontiguousarray(a, np.float32) for a in (pre, g, beta))
    state, conv = np.array(state, np.float32, order="C"), np.array(conv, np.float32, order="C")
    M, Cc = pre.shape
    post, core = np.zeros((M, Cc), np.float32), np.zeros((M, HV * Dv), np.float32)
    check(lib().ling_b200_gdn_prefill_host(device, Hk, HV, Dk, Dv, M, _fp(pre), _u16(convw_bits), _fp(g), _fp(beta), _fp(state), _fp(conv),
                                           _fp(post), _fp(core)), "gdn_prefill")
    return post, core, state, conv


def gdn_chunk_bench(Hk, HV, M, iters=10, device=0):
    ms = C.c_float()
    check(lib().ling_b200_gdn_chunk_bench(device, Hk, HV, M, iters, C.byref(ms)), "gdn_chunk_bench")
    return ms.value


class PrefillGdnLayer:
    """One DeltaNet layer's mixer on the prefill path with synthetic weights (ling_b200_prefill_gdn_*)."""

    def __init__(self, hidden, k_heads, v_heads, max_rows, seed=0, device=0):
        self.H, self.Hk, self.HV, self.max_rows = hidden, k_heads, v_heads, max_rows
        self.C, self.Vs = (2 * k_heads + v_heads) * 128, v_heads * 128
        self.h = C.c_void_p()
        check(lib().ling_b200_prefill_gdn_create(device, hidden, k_heads, v_heads, max_rows, C.c_uint64(seed), C.byref(self.h)), "prefill_gdn_create")

    def close(self):
        if self.h:
            lib().ling_b200_prefill_gdn_destroy(self.h)
            self.h = C.c_void_p()

    def set_state(self, state=None, conv=None):
        s = None if state is None else np.ascontiguousarray(state, np.float32)
        c = None if conv is None else np.ascontiguousarray(conv, np.float32)
        check(lib().ling_b200_prefill_gdn_state(self.h, 1, None if s is None else _fp(s), None if c is None else _fp(c)), "prefill_gdn_state")

    def get_state(self):
        s, c = np.zeros((self.HV, 128, 128), np.float32), np.zeros((self.C, 3), np.float32)
        check(lib().ling_b200_prefill_gdn_state(self.h, 0, _fp(s), _fp(c)), "prefill_gdn_state")
        return s, c

    def forward(self, h):
        h = np.ascontiguousarray(h, np.float32)
        out = np.zeros_like(h)
        check(lib().ling_b200_prefill_gdn_forward(self.h, _fp(h), h.shape[0], _fp(out)), "prefill_gdn_forward")
        return out

    def bench(self, rows, repeats=3):
        ms = C.c_float()
        check(lib().ling_b200_prefill_gdn_bench(self.h, rows, repeats, C.byref(ms)), "prefill_gdn_bench")
        return ms.value / repeats

    def stages(self, rows):
        o = {"xn": np.zeros((rows, self.H), np.float32), "pre": np.zeros((rows, self.C), np.float32), "z": np.zeros((rows, self.Vs), np.float32),
             "g": np.zeros((rows, self.HV), np.float32), "beta": np.zeros((rows, self.HV), np.float32), "core": np.zeros((rows, self.Vs), np.float32)}
        check(lib().ling_b200_prefill_gdn_read_stages(self.h, rows, *[_fp(o[k]) for k in ("xn", "pre", "z", "g", "beta", "core")]), "read_stages")
        return o

    def weights(self):
        H, Cc, Vs, HV = self.H, self.C, self.Vs, self.HV
        w = {"norm": np.zeros(H, np.uint16), "convw": np.zeros((Cc, 4), np.uint16), "wa": np.zeros((HV, H), np.uint16), "wb": np.zeros((HV, H), np.uint16),
             "A_log": np.zeros(HV, np.uint16), "dt_bias": np.zeros(HV, np.uint16), "lin_norm": np.zeros(128, np.uint16),
             "qkv_q": np.zeros((Cc, H // 2), np.uint8), "qkv_s": np.zeros((Cc, H // 16), np.uint8), "z_q": np.zeros((Vs, H // 2), np.uint8),
             "z_s": np.zeros((Vs, H // 16), np.uint8), "out_q": np.zeros((H, Vs // 2), np.uint8), "out_s": np.zeros((H, Vs // 16), np.uint8)}
        sc = np.zeros(5, np.float32)
        check(lib().ling_b200_prefill_gdn_read_weights(self.h, *[_u16(w[k]) for k in ("norm", "convw", "wa", "wb", "A_log", "dt_bias", "lin_norm")],
                                                       *[_bp(w[k]) for k in ("qkv_q", "qkv_s", "z_q", "z_s", "out_q", "out_s")], _fp(sc)), "read_weights")
        w["in_scale"], w["mid_scale"], w["s_qkv"], w["s_z"], w["s_out"] = (float(v) for v in sc)
        return w


def topk_rows(x, k, device=0):
    """Per row the k largest values, descending, ties to the lower index (ling_b200_topk_rows_host)."""
    x = np.ascontiguousarray(x, np.float32)
    vals, ids = np.zeros((x.shape[0], k), np.float32), np.zeros((x.shape[0], k), np.int32)
    check(lib().ling_b200_topk_rows_host(device, _fp(x), x.shape[0], x.shape[1], k, _fp(vals), _ip(ids)), "topk_rows")
    return vals, ids


def _u16(a):
    return a.ctypes.data_as(C.POINTER(C.c_uint16))


def selector_lattice(cand, unary, pred_bits, succ_bits, anchor, hp=None, x=None, proj_bits=None, device=0):
    """The candidate selector's 16 x 16 scores per position; with x and proj_bits the projection hp = x . proj^T is computed
    first (returned as the second value).  Codebooks and projection as BF16 bit patterns (to_bf16_bits)."""
    cand, unary = np.ascontiguousarray(cand, np.int32), np.ascontiguousarray(unary, np.float32)
    E, vocab = cand.shape[0], pred_bits.shape[0]
    scores = np.zeros((E, 16, 16), np.float32)
    if x is not None:
        x = np.ascontiguousarray(x, np.float32)
        hp = np.zeros((E, 256), np.float32)
        check(lib().ling_b200_selector_lattice_host(device, _fp(x), _u16(proj_bits), x.shape[1], _fp(hp), _ip(cand), _fp(unary),
                                                    _u16(pred_bits), _u16(succ_bits), vocab, int(anchor), E, _fp(scores)), "selector_lattice")
    else:
        hp = np.ascontiguousarray(hp, np.float32)
        check(lib().ling_b200_selector_lattice_host(device, None, None, 0, _fp(hp), _ip(cand), _fp(unary), _u16(pred_bits),
                                                    _u16(succ_bits), vocab, int(anchor), E, _fp(scores)), "selector_lattice")
    return scores, hp


def sparse_select(p, us_bits, masks, dynamic, cap, device=0):
    """The sparse head's selection (ling_b200_sparse_select_host): p [M][256], us_bits [N][256] BF16 bits, masks [n][N] bytes.
    Returns (rows ascending, keys [N] uint32: what the selection ranked, 0 = marked)."""
    p = np.ascontiguousarray(p, np.float32)
    us_bits = np.ascontiguousarray(us_bits, np.uint16)
    masks = np.ascontiguousarray(np.atleast_2d(masks), np.uint8)
    N = us_bits.shape[0]
    rows, n, keys = np.zeros(cap, np.int32), C.c_int(0), np.zeros(N, np.uint32)
    check(lib().ling_b200_sparse_select_host(device, _fp(p), p.shape[0], _u16(us_bits), N, _bp(masks), masks.shape[0], dynamic, cap,
                                             _ip(rows), C.byref(n), keys.ctypes.data_as(C.POINTER(C.c_uint32))), "sparse_select")
    return rows[:n.value].copy(), keys


def sparse_select_bench(N, M, dynamic, cap, iters=20, device=0):
    """(ms of the scores kernel alone, ms of the whole selection) on synthetic factors resident in HBM."""
    ms = (C.c_float * 2)()
    check(lib().ling_b200_sparse_select_bench(device, N, M, dynamic, cap, iters, ms), "sparse_select_bench")
    return ms[0], ms[1]


class DraftHead:
    """The drafter's last stage on a Context (ling_b200_draft_head_*): rows after the drafter's final norm in, candidates and
    selector scores out."""

    def __init__(self, ctx, proj_bits, pred_bits, succ_bits):
        self.ctx, self.h = ctx, C.c_void_p()
        check(lib().ling_b200_draft_head_create(ctx.h, _u16(proj_bits), _u16(pred_bits), _u16(succ_bits), C.byref(self.h)), "draft_head_create")

    def run(self, x, anchor):
        x = np.ascontiguousarray(x, np.float32)
        E = x.shape[0]
        cand, unary, scores = np.zeros((E, 16), np.int32), np.zeros((E, 16), np.float32), np.zeros((E, 16, 16), np.float32)
        check(lib().ling_b200_draft_head_run(self.h, _fp(x), E, int(anchor), _ip(cand), _fp(unary), _fp(scores)), "draft_head_run")
        return cand, unary, scores

    def enable_sparse(self, us_bits, vt_bits, dynamic, cap):
        """The sparse head: us [vocab][256] and vt [256][hidden] BF16 bits (the head's rank-256 factors)."""
        check(lib().ling_b200_draft_head_enable_sparse(self.h, _u16(np.ascontiguousarray(us_bits, np.uint16)),
                                                       _u16(np.ascontiguousarray(vt_bits, np.uint16)), dynamic, cap), "draft_head_enable_sparse")
        self.cap = cap

    def mask_reset(self, session, ids):
        ids = np.ascontiguousarray(ids, np.int32)
        check(lib().ling_b200_draft_head_mask_reset(self.h, session, _ip(ids), len(ids)), "draft_head_mask_reset")

    def mask_mark(self, session, ids):
        ids = np.ascontiguousarray(ids, np.int32)
        check(lib().ling_b200_draft_head_mask_mark(self.h, session, _ip(ids), len(ids)), "draft_head_mask_mark")

    def run_sparse(self, session, x, anchor):
        """As run, scoring only the session's mask and the rows the rank-256 factors rate best; also returns the scored rows."""
        x = np.ascontiguousarray(x, np.float32)
        E = x.shape[0]
        cand, unary, scores = np.zeros((E, 16), np.int32), np.zeros((E, 16), np.float32), np.zeros((E, 16, 16), np.float32)
        n, sel = C.c_int(0), np.zeros(self.cap, np.int32)
        check(lib().ling_b200_draft_head_run_sparse(self.h, session, _fp(x), E, int(anchor), _ip(cand), _fp(unary), _fp(scores), C.byref(n),
                                                    _ip(sel)), "draft_head_run_sparse")
        return cand, unary, scores, sel[:n.value].copy()

    def close(self):
        if self.h:
            lib().ling_b200_draft_head_destroy(self.h)
            self.h = C.c_void_p()


def describe_tree(parent, chain):
    par = np.ascontiguousarray(parent, np.int32)
    t = TreeDesc()
    rc = lib().ling_b200_describe_tree(_ip(par), len(par), chain, C.byref(t))
    return rc, t
