"""TEST INFRASTRUCTURE: ctypes bindings of the CPU oracle.

`port()` is oracle/libjasmine_oracle.so, the restatement; `ref()` is
oracle/_ref/libjasmine_ref.so, the reference's own headers behind C entry
points (None when it was not built).  Arrays are float32 / int32 numpy arrays,
row-major.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
ORACLE_DIR = ROOT / "oracle"
_fp = C.POINTER(C.c_float)
_ip = C.POINTER(C.c_int)
_port = None
_ref = None


def build() -> None:
    """Compile the oracle (and oracle/_ref when the reference sources are present)."""
    subprocess.run(["make", "-C", str(ORACLE_DIR)], check=True, capture_output=True)


def port() -> C.CDLL:
    global _port
    if _port is None:
        so = ORACLE_DIR / "libjasmine_oracle.so"
        if not so.exists():
            build()
        _port = C.CDLL(str(so))
        for name in ("orc_mha_weight_count", "orc_encoder_weight_count", "orc_gpt_weight_count"):
            getattr(_port, name).restype = C.c_long
    return _port


def ref():
    global _ref
    if _ref is None:
        so = ORACLE_DIR / "_ref" / "libjasmine_ref.so"
        if not so.exists():
            return None
        _ref = C.CDLL(str(so))
        for name in ("ref_mha_weight_count", "ref_encoder_weight_count", "ref_gpt_weight_count"):
            getattr(_ref, name).restype = C.c_long
    return _ref


def f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def P(a):
    return None if a is None else a.ctypes.data_as(_fp)


def PI(a):
    return None if a is None else a.ctypes.data_as(_ip)


def cf(x) -> C.c_float:
    return C.c_float(float(x))


class Oracle:
    """The same call surface over either library (prefix 'orc' or 'ref')."""

    def __init__(self, lib, prefix: str):
        self.lib, self.prefix = lib, prefix

    def _f(self, name):
        return getattr(self.lib, f"{self.prefix}_{name}")

    def expr(self, op, A, B=None, s=0.0):
        A = f32(A)
        R, Cc = A.shape
        if B is not None:
            B = f32(B)
            Br, Bc = B.shape
        else:
            Br = Bc = 1
        out = np.empty((max(R, Br) if op != 12 else R, max(Cc, Bc) if op != 12 else Cc), np.float32)
        rc = self._f("expr")(op, P(A), R, Cc, P(B), Br, Bc, cf(s), P(out))
        assert rc == 0, rc
        return out

    def reduce(self, kind, A):
        A = f32(A)
        R, Cc = A.shape
        n = {0: R, 1: R, 2: R, 3: Cc, 4: Cc}.get(kind, 1)
        out = np.empty(n, np.float32)
        assert self._f("reduce")(kind, P(A), R, Cc, P(out)) == 0
        return out

    def hsoftmax(self, A, B=None, s=1.0):
        A = f32(A)
        out = np.empty_like(A)
        assert self._f("hsoftmax")(P(A), P(f32(B)) if B is not None else None, cf(s), A.shape[0], A.shape[1], P(out)) == 0
        return out

    def softmax_full(self, A):
        A = f32(A)
        out = np.empty_like(A)
        assert self._f("softmax_full")(P(A), A.shape[0], A.shape[1], P(out)) == 0
        return out

    # token-major [T, d] in and out for both libraries (the reference works on the transpose)
    def layer_norm(self, x, x2=None, gain=None, bias=None, eps=0.0):
        x = f32(x)
        T, d = x.shape
        out = np.empty_like(x)
        if self.prefix == "orc":
            assert self.lib.orc_layer_norm_rows(P(x), P(f32(x2)) if x2 is not None else None, T, d,
                                                P(f32(gain)) if gain is not None else None,
                                                P(f32(bias)) if bias is not None else None, cf(eps), P(out)) == 0
            return out
        xt = f32(x.T)
        ot = np.empty_like(xt)
        if gain is None and bias is None and eps == 0.0 and x2 is None:
            assert self.lib.ref_layer_norm(P(xt), d, T, P(ot)) == 0
        else:
            g = f32(gain if gain is not None else np.ones(d))
            b = f32(bias if bias is not None else np.zeros(d))
            x2t = f32(x2.T) if x2 is not None else None
            assert self.lib.ref_layer_norm_eps(P(xt), P(x2t), d, T, P(g), P(b), cf(eps), P(ot)) == 0
        return f32(ot.T)

    def rms_norm(self, x, gain, eps):
        x = f32(x)
        T, d = x.shape
        if self.prefix == "orc":
            out = np.empty_like(x)
            assert self.lib.orc_rms_norm_rows(P(x), T, d, P(f32(gain)), cf(eps), P(out)) == 0
            return out
        xt = f32(x.T)
        ot = np.empty_like(xt)
        assert self.lib.ref_rms_norm(P(xt), d, T, P(f32(gain)), cf(eps), P(ot)) == 0
        return f32(ot.T)

    def dot(self, A, B):
        A, B = f32(A), f32(B)
        out = np.empty((A.shape[0], B.shape[1]), np.float32)
        rc = self._f("dot")(P(A), A.shape[0], A.shape[1], P(B), B.shape[0], B.shape[1], P(out))
        return rc, out

    def linear(self, X, W, b):
        """X:[T,K] token-major, W:[N,K], b:[N] -> [T,N]  (weight_net_t::forward on the transpose)."""
        X, W, b = f32(X), f32(W), f32(b)
        T, K = X.shape
        N = W.shape[0]
        if self.prefix == "orc":
            out = np.empty((T, N), np.float32)
            assert self.lib.orc_linear(P(X), P(W), P(b), T, N, K, P(out)) == 0
            return out
        w = f32(np.concatenate([W.ravel(), b.ravel()]))
        xt = f32(X.T)
        yt = np.empty((N, T), np.float32)
        assert self.lib.ref_weight_net(P(w), K, N, P(xt), T, P(yt)) == 0
        return f32(yt.T)

    def activation(self, kind, X):
        X = f32(X)
        out = np.empty_like(X)
        if self.prefix == "orc":
            assert self.lib.orc_activation(kind, P(X), C.c_long(X.size), P(out)) == 0
        else:
            assert self.lib.ref_activation(kind, P(X), X.shape[0], X.shape[1], P(out)) == 0
        return out

    def mha_weight_count(self, H, d):
        return int(self._f("mha_weight_count")(H, d))

    def mha(self, w, x, H, causal):
        """x: [T, d] token-major."""
        x, w = f32(x), f32(w)
        T, d = x.shape
        if self.prefix == "orc":
            out = np.empty_like(x)
            rc = self.lib.orc_mha(P(w), P(x), T, H, d, int(causal), P(out))
            assert rc == 0, rc
            return out
        xt = f32(x.T)
        ot = np.empty_like(xt)
        assert self.lib.ref_mha(P(w), P(xt), H, d, T, int(causal), P(ot)) == 0
        return f32(ot.T)

    def rope(self, x):
        """reference-mode RoPE over the whole feature vector; x: [T, d] token-major."""
        x = f32(x)
        T, d = x.shape
        if self.prefix == "orc":
            table = np.empty((T, d // 2, 4), np.float32)
            assert self.lib.orc_rope_table(0, d, cf(10000.0), T, P(table)) == 0
            out = np.empty_like(x)
            assert self.lib.orc_rope_apply(P(x), P(out), P(table), d, 1, None, T) == 0
            return out
        xt = f32(x.T)
        ot = np.empty_like(xt)
        assert self.lib.ref_rope(P(xt), d, T, P(ot)) == 0
        return f32(ot.T)

    def encoder_weight_count(self, L, H, d):
        return int(self._f("encoder_weight_count")(L, H, d))

    def encoder(self, w, x, L, H, causal, rope):
        x, w = f32(x), f32(w)
        T, d = x.shape
        if self.prefix == "orc":
            out = np.empty_like(x)
            assert self.lib.orc_encoder(P(w), P(x), L, H, d, T, int(causal), int(rope), P(out)) == 0
            return out
        xt = f32(x.T)
        ot = np.empty_like(xt)
        assert self.lib.ref_encoder(P(w), P(xt), L, H, d, T, int(causal), int(rope), P(ot)) == 0
        return f32(ot.T)

    def gpt_weight_count(self, L, d, H, ffn, vocab, max_pos):
        return int(self._f("gpt_weight_count")(L, d, H, ffn, vocab, max_pos))

    def gpt(self, w, L, d, H, ffn, vocab, max_pos, eps, ids, n_gen, want_gen_logits=True):
        w = f32(w)
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        S = ids.shape[0]
        logits = np.empty((S, vocab), np.float32)
        gen = np.zeros(max(n_gen, 1), np.int32)
        gl = np.empty((max(n_gen, 1), vocab), np.float32) if want_gen_logits else None
        rc = self._f("gpt")(P(w), L, d, H, ffn, vocab, max_pos, cf(eps), PI(ids), S, P(logits), n_gen, PI(gen), P(gl))
        assert rc == 0, rc
        return logits, gen[:n_gen], (gl[:n_gen] if gl is not None else None)


def port_oracle() -> Oracle:
    return Oracle(port(), "orc")


def ref_oracle():
    r = ref()
    return Oracle(r, "ref") if r is not None else None


# ---- functions only the port has -----------------------------------------------------------
def rope_table(mode, d, theta, max_pos):
    t = np.empty((max_pos, d // 2, 4), np.float32)
    assert port().orc_rope_table(mode, d, cf(theta), max_pos, P(t)) == 0
    return t


def rope_apply(x, table, d, n_heads, positions=None):
    x = f32(x)
    out = np.empty_like(x)
    pos = np.ascontiguousarray(positions, dtype=np.int32) if positions is not None else None
    assert port().orc_rope_apply(P(x), P(out), P(f32(table)), d, n_heads, PI(pos), x.shape[0]) == 0
    return out


def attention(q, k, v, batch, Hq, Hkv, D, causal, scale=None, exact_div=True):
    q, k, v = f32(q), f32(k), f32(v)
    Tq, Tk = q.shape[0] // batch, k.shape[0] // batch
    out = np.empty_like(q)
    scale = float(D) ** -0.5 if scale is None else scale
    assert port().orc_attention(P(q), P(k), P(v), P(out), batch, Tq, Tk, Hq, Hkv, D, int(causal), cf(scale), int(exact_div)) == 0
    return out


def fill(n, seed, tensor_id, dist, a, b, to_bf16=False):
    out = np.empty(n, np.float32)
    assert port().orc_fill(P(out), C.c_long(n), C.c_uint64(seed), C.c_uint64(tensor_id), dist, cf(a), cf(b), int(to_bf16)) == 0
    return out


class LlamaCfg(C.Structure):
    _fields_ = [("L", C.c_int), ("d", C.c_int), ("Hq", C.c_int), ("Hkv", C.c_int), ("D", C.c_int), ("ffn", C.c_int),
                ("vocab", C.c_int), ("eps", C.c_float), ("theta", C.c_float)]


def llama_forward(cfg: dict, emb, layers, gf, wlm, ids, round_act=True, last_rows=0):
    """layers: list of 9-tuples (g1, wq, wk, wv, wo, g2, wgate, wup, wdown) of float32 arrays.
    last_rows > 0: only the logits of the last `last_rows` tokens are computed (the other rows of the result are
    meaningless) - the lm_head over every prompt position is most of the work at a 32000-word vocabulary."""
    c = LlamaCfg(cfg["L"], cfg["d"], cfg["Hq"], cfg["Hkv"], cfg["D"], cfg["ffn"], cfg["vocab"], cfg["eps"], cfg["theta"])
    keep = [f32(a) for lw in layers for a in lw]
    ptrs = (_fp * len(keep))(*[P(a) for a in keep])
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    T = ids.shape[0]
    logits = np.empty((T, cfg["vocab"]), np.float32)
    emb, gf, wlm = f32(emb), f32(gf), f32(wlm)
    assert port().orc_llama_forward(C.byref(c), P(emb), ptrs, P(gf), P(wlm), PI(ids), T, int(round_act), P(logits), int(last_rows)) == 0
    return logits
