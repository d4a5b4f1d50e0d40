"""ctypes front end of the CPU checker `librnnt_oracle.so` plus an independent brute-force path enumerator.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke test and by bench.py's CPU-baseline / reference legs.
The product package never imports this module.
"""
import ctypes
import itertools
import math
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "librnnt_oracle.so")
_lib = None

_i32p = ctypes.POINTER(ctypes.c_int32)
_i64p = ctypes.POINTER(ctypes.c_int64)
_f64p = ctypes.POINTER(ctypes.c_double)
_f32p = ctypes.POINTER(ctypes.c_float)


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "rnnt_oracle.c")
    if force or not os.path.isfile(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "librnnt_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


def lib():
    global _lib
    if _lib is None:
        if not os.path.isfile(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
        _lib.oracle_offsets.restype = ctypes.c_int64
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def _p(a, typ):
    return None if a is None else a.ctypes.data_as(typ)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def num_threads() -> int:
    return lib().oracle_num_threads()


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(int(n))


def offsets(lx, ly):
    lx, ly = _c(lx, np.int32), _c(ly, np.int32)
    off = np.zeros(max(len(lx), 1), dtype=np.int64)
    rows = lib().oracle_offsets(_p(lx, _i32p), _p(ly, _i32p), ctypes.c_int64(len(lx)), _p(off, _i64p))
    return off[:len(lx)], int(rows)


def log_softmax(x):
    x = _c(x, np.float64)
    out = np.empty_like(x)
    lib().oracle_log_softmax_f64(_p(x, _f64p), ctypes.c_int64(x.shape[0]), ctypes.c_int64(x.shape[1]), _p(out, _f64p))
    return out


def gather(lp, lx, ly, y, blank):
    lp, lx, ly, y = _c(lp, np.float64), _c(lx, np.int32), _c(ly, np.int32), _c(y, np.int32)
    y = y.reshape(len(lx), -1)
    off, rows = offsets(lx, ly)
    assert rows == lp.shape[0], (rows, lp.shape)
    out = np.zeros((rows, 2), dtype=np.float64)
    lib().oracle_gather_f64(_p(lp, _f64p), ctypes.c_int64(lp.shape[1]), _p(lx, _i32p), _p(ly, _i32p), _p(y, _i32p),
                            ctypes.c_int64(y.shape[1]), ctypes.c_int64(len(lx)), _p(off, _i64p),
                            ctypes.c_int32(blank), _p(out, _f64p))
    return out


def forward(g, lx, ly, want_grads=True, want_ab=False):
    """Reference forward on gathered log-probs [STU,2] in double. Returns dict(costs, grads, alpha, beta, mismatch)."""
    g, lx, ly = _c(g, np.float64), _c(lx, np.int32), _c(ly, np.int32)
    off, rows = offsets(lx, ly)
    assert rows == g.shape[0]
    N = len(lx)
    costs = np.zeros(N)
    grads = np.zeros((rows, 2)) if want_grads else None
    alpha = np.zeros(rows) if want_ab else None
    beta = np.zeros(rows) if want_ab else None
    mism = np.zeros(N, dtype=np.int32)
    lib().oracle_forward_f64(_p(g, _f64p), _p(lx, _i32p), _p(ly, _i32p), ctypes.c_int64(N), _p(off, _i64p),
                             _p(costs, _f64p), _p(grads, _f64p), _p(alpha, _f64p), _p(beta, _f64p), _p(mism, _i32p))
    return dict(costs=costs, grads=grads, alpha=alpha, beta=beta, mismatch=mism, offset=off)


def forward_ref32(g, lx, ly, want_ab=False):
    """Reference forward in the float arithmetic the reference uses for float32 inputs."""
    g, lx, ly = _c(g, np.float32), _c(lx, np.int32), _c(ly, np.int32)
    off, rows = offsets(lx, ly)
    assert rows == g.shape[0]
    N = len(lx)
    costs = np.zeros(N, dtype=np.float32)
    grads = np.zeros((rows, 2), dtype=np.float32)
    alpha = np.zeros(rows, dtype=np.float32) if want_ab else None
    beta = np.zeros(rows, dtype=np.float32) if want_ab else None
    lib().oracle_forward_ref32(_p(g, _f32p), _p(lx, _i32p), _p(ly, _i32p), ctypes.c_int64(N), _p(off, _i64p),
                               _p(costs, _f32p), _p(grads, _f32p), _p(alpha, _f32p), _p(beta, _f32p))
    return dict(costs=costs, grads=grads, alpha=alpha, beta=beta, offset=off)


def costs_only(g, lx, ly):
    g, lx, ly = _c(g, np.float64), _c(lx, np.int32), _c(ly, np.int32)
    off, rows = offsets(lx, ly)
    costs = np.zeros(len(lx))
    lib().oracle_costs_f64(_p(g, _f64p), _p(lx, _i32p), _p(ly, _i32p), ctypes.c_int64(len(lx)), _p(off, _i64p),
                           _p(costs, _f64p))
    return costs


def backward(grads, grad_costs, lx, ly, y, blank, V, accumulate_equal=False):
    grads, gc = _c(grads, np.float64), _c(grad_costs, np.float64)
    lx, ly, y = _c(lx, np.int32), _c(ly, np.int32), _c(y, np.int32).reshape(len(lx), -1)
    off, rows = offsets(lx, ly)
    dense = np.zeros((rows, V))
    lib().oracle_backward_f64(_p(grads, _f64p), _p(gc, _f64p), _p(lx, _i32p), _p(ly, _i32p), _p(y, _i32p),
                              ctypes.c_int64(y.shape[1]), ctypes.c_int64(len(lx)), _p(off, _i64p),
                              ctypes.c_int32(blank), ctypes.c_int64(V), ctypes.c_int(int(accumulate_equal)),
                              _p(dense, _f64p))
    return dense


def fused(x, lx, ly, y, blank, weights=None, want_grad=True):
    """log_softmax -> transducer loss -> gradient w.r.t. the logits, all in double. Returns (costs[N], dense|None)."""
    x, lx, ly = _c(x, np.float64), _c(lx, np.int32), _c(ly, np.int32)
    y = _c(y, np.int32).reshape(len(lx), -1)
    N = len(lx)
    costs = np.zeros(N)
    dense = np.zeros_like(x) if want_grad else None
    w = None if weights is None else _c(weights, np.float64)
    lib().oracle_fused_f64(_p(x, _f64p), ctypes.c_int64(x.shape[1]), _p(lx, _i32p), _p(ly, _i32p), _p(y, _i32p),
                           ctypes.c_int64(y.shape[1]), ctypes.c_int64(N), ctypes.c_int32(blank), _p(w, _f64p),
                           _p(costs, _f64p), _p(dense, _f64p))
    return costs, dense


def fused_f32io(x, lx, ly, y, blank, weights=None, want_grad=True, dense_out=None):
    """Float32 in / float32 gradient out flavour used as the timed CPU baseline."""
    x, lx, ly = _c(x, np.float32), _c(lx, np.int32), _c(ly, np.int32)
    y = _c(y, np.int32).reshape(len(lx), -1)
    N = len(lx)
    costs = np.zeros(N)
    dense = None
    if want_grad:
        dense = dense_out if dense_out is not None else np.empty_like(x)
    w = None if weights is None else _c(weights, np.float64)
    lib().oracle_fused_f32io(_p(x, _f32p), ctypes.c_int64(x.shape[1]), _p(lx, _i32p), _p(ly, _i32p), _p(y, _i32p),
                             ctypes.c_int64(y.shape[1]), ctypes.c_int64(N), ctypes.c_int32(blank), _p(w, _f64p),
                             _p(costs, _f64p), _p(dense, _f32p))
    return costs, dense


def viterbi(g, lx, ly):
    """Best path of every sequence from gathered log-probs [STU,2] in double. Returns (moves [N, max(T+U)] int32 -
    0 = blank move, 1 = label move, -1 beyond T_n+U_n - and the paths' log-probabilities [N])."""
    g, lx, ly = _c(g, np.float64), _c(lx, np.int32), _c(ly, np.int32)
    off, rows = offsets(lx, ly)
    assert rows == g.shape[0]
    N = len(lx)
    stride = int((lx.astype(np.int64) + ly).max()) if N else 0
    moves = np.zeros((N, stride), dtype=np.int32)
    scores = np.zeros(N)
    lib().oracle_viterbi_f64(_p(g, _f64p), _p(lx, _i32p), _p(ly, _i32p), ctypes.c_int64(N), _p(off, _i64p),
                             ctypes.c_int64(stride), _p(moves, _i32p), _p(scores, _f64p))
    return moves, scores


def posteriors(g, lx, ly):
    """exp(alpha + beta - log P) of every lattice node, compact [STU] in (t,u) row-major order per sequence."""
    g, lx, ly = _c(g, np.float64), _c(lx, np.int32), _c(ly, np.int32)
    off, rows = offsets(lx, ly)
    assert rows == g.shape[0]
    post = np.zeros(rows)
    lib().oracle_posteriors_f64(_p(g, _f64p), _p(lx, _i32p), _p(ly, _i32p), ctypes.c_int64(len(lx)), _p(off, _i64p),
                                _p(post, _f64p))
    return post


# ---------------------------------------------------------------- independent brute force (tiny lattices only)

def brute_force_best_path(lp_blank, lp_label):
    """(log-probability, moves) of the most probable monotone path through a T x (U+1) lattice, by enumeration; moves
    as in `viterbi` (the final blank included). Ties: the path whose label moves come latest, which is what a
    recursion that prefers the blank move on equal scores walks back to... only when no tie occurs is the path
    unique, so callers compare scores, and paths only on inputs without ties (random reals)."""
    T, m = len(lp_blank), len(lp_blank[0])
    U = m - 1
    best, best_moves = -math.inf, None
    for labels_at in itertools.combinations(range(T - 1 + U), U):
        t = u = 0
        logp = 0.0
        pos = set(labels_at)
        for step in range(T - 1 + U):
            if step in pos:
                logp += lp_label[t][u]
                u += 1
            else:
                logp += lp_blank[t][u]
                t += 1
        logp += lp_blank[T - 1][U]
        if logp > best:
            best, best_moves = logp, [1 if k in pos else 0 for k in range(T - 1 + U)] + [0]
    return best, best_moves


def brute_force_cost(lp_blank, lp_label):
    """-log of the summed probability of every monotone path through a T x (U+1) lattice.

    lp_blank[t][u], lp_label[t][u] are log-probabilities of the blank / label move out of cell (t,u). A path makes
    U label moves and T blank moves, the last move being the blank out of (T-1,U). Exponential cost: T+U <= ~14.
    """
    T, m = len(lp_blank), len(lp_blank[0])
    U = m - 1
    total = 0.0
    for labels_at in itertools.combinations(range(T - 1 + U), U):
        t = u = 0
        logp = 0.0
        pos = set(labels_at)
        for step in range(T - 1 + U):
            if step in pos:
                logp += lp_label[t][u]
                u += 1
            else:
                logp += lp_blank[t][u]
                t += 1
        assert t == T - 1 and u == U
        logp += lp_blank[T - 1][U]
        total += math.exp(logp)
    return -math.log(total)


_ACT = {
    None: (lambda s: s, lambda s: np.ones_like(s)),
    "none": (lambda s: s, lambda s: np.ones_like(s)),
    "relu": (lambda s: np.maximum(s, 0.0), lambda s: (s > 0).astype(s.dtype)),
    "tanh": (np.tanh, lambda s: 1.0 - np.tanh(s) ** 2),
}


def joint_compact(enc, pred, lx, ly, activation="tanh"):
    """act(enc[n, t] + pred[n, u]) for every lattice node in the compact layout of the reference's test
    (test/test.py:34-48: sequence n contributes its [:T_n, :U_n+1] block, rows in (t, u) order). Double precision.
    enc [B, t_max, H], pred [B, u_max1, H] -> [sum_n T_n (U_n+1), H]."""
    act, _ = _ACT[activation]
    enc, pred = np.asarray(enc, np.float64), np.asarray(pred, np.float64)
    rows = []
    for n in range(len(lx)):
        T, m = int(lx[n]), int(ly[n]) + 1
        rows.append(act(enc[n, :T, None, :] + pred[n, None, :m, :]).reshape(T * m, -1))
    return np.concatenate(rows, axis=0) if rows else np.zeros((0, enc.shape[2]))


def joint_compact_backward(enc, pred, lx, ly, grad_out, activation="tanh"):
    """Gradients of joint_compact w.r.t. enc and pred (zero in the padding), double precision."""
    _, slope = _ACT[activation]
    enc, pred = np.asarray(enc, np.float64), np.asarray(pred, np.float64)
    g = np.asarray(grad_out, np.float64)
    genc, gpred = np.zeros_like(enc), np.zeros_like(pred)
    at = 0
    for n in range(len(lx)):
        T, m = int(lx[n]), int(ly[n]) + 1
        s = enc[n, :T, None, :] + pred[n, None, :m, :]
        d = g[at:at + T * m].reshape(T, m, -1) * slope(s)
        genc[n, :T] = d.sum(axis=1)
        gpred[n, :m] = d.sum(axis=0)
        at += T * m
    return genc, gpred
