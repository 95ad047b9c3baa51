"""Python front end of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the CPU-baseline / reference legs of the
benchmark may import this module; the product package never does.

Three independent checkers live here:

* :func:`oracle_loss` - the C restatement (``transducer_oracle.c``) of the
  reference's CPU algorithm (optimized_transducer/csrc/cpu.cc), in float32 or
  float64, through ctypes.
* :func:`brute_force_score` - path enumeration on tiny lattices, for both the
  standard and the one-symbol-per-frame recursion.  It shares no code with the
  recursions, so it pins them independently of the reference.
* :func:`ref_loss` / :func:`ref_stages` - the reference's own CPU build
  (``oracle/_ref``, produced by ``build_ref.py``), when it has been built.
"""
import ctypes
import importlib.machinery
import importlib.util
import itertools
import math
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = {}


def build_oracle():
    """Runs ``make`` in this directory (gcc only)."""
    subprocess.run(["make", "-C", HERE], check=True, capture_output=True)
    return os.path.join(HERE, "libot_oracle.so")


def _lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(HERE, "libot_oracle.so")
        if not os.path.isfile(path):
            build_oracle()
        lib = ctypes.CDLL(path)
        p = ctypes.c_void_p
        for name, real in (("ot_oracle_loss_f32", ctypes.c_float),
                           ("ot_oracle_loss_f64", ctypes.c_double)):
            fn = getattr(lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [p, p, p, p, p, ctypes.c_int32, ctypes.c_int32,
                           ctypes.c_int32, ctypes.c_int32, ctypes.c_int,
                           ctypes.c_int, real, p, p, p, p, p, p]
        lib.ot_oracle_set_threads.restype = ctypes.c_int
        lib.ot_oracle_set_threads.argtypes = [ctypes.c_int]
        _LIB = lib
    return _LIB


def set_threads(n):
    """Sets the OpenMP thread count of the C oracle; returns the count in use."""
    return _lib().ot_oracle_set_threads(int(n))


def row_splits(T, U):
    """Exclusive prefix sum of T_b * (U_b + 1): first packed row of each utterance."""
    cells = np.asarray(T, np.int64) * (np.asarray(U, np.int64) + 1)
    return np.concatenate([[0], np.cumsum(cells)])


def oracle_loss(x, targets, T, U, blank, from_log_softmax=False,
                one_sym_per_frame=False, want_grad=True, fill=np.nan,
                in_place=False):
    """Runs the C oracle.

    ``x`` is the packed (rows, V) array; its dtype (float32 / float64) selects
    the precision.  Returns a dict with ``scores`` (log-likelihood per
    utterance, from the alpha side), ``scores_beta``, ``den`` (None when
    ``from_log_softmax``), ``lp`` (rows, 2), ``alpha``, ``beta`` (rows) and
    ``grad`` ((rows, V) or None).  Off-band cells of alpha/beta in the modified
    recursion hold ``fill``.  With ``in_place`` the gradient overwrites ``x``.
    """
    x = np.ascontiguousarray(x)
    assert x.dtype in (np.float32, np.float64) and x.ndim == 2
    dt = x.dtype
    targets = np.ascontiguousarray(targets, np.int32)
    T = np.ascontiguousarray(T, np.int32)
    U = np.ascontiguousarray(U, np.int32)
    N, V = int(T.shape[0]), int(x.shape[1])
    assert targets.ndim == 2 and targets.shape[0] == N
    rows = int(row_splits(T, U)[-1])
    assert rows == x.shape[0], (rows, x.shape)
    max_u = max(int(targets.shape[1]), 1)
    if targets.shape[1] == 0:
        targets = np.zeros((N, 1), np.int32)
    den = None if from_log_softmax else np.empty(rows, dt)
    lp = np.empty((rows, 2), dt)
    alpha = np.empty(rows, dt)
    beta = np.empty(rows, dt)
    sa = np.empty(N, dt)
    sb = np.empty(N, dt)
    grad = None
    if want_grad:
        grad = x if in_place else np.empty_like(x)

    def ptr(a):
        return None if a is None else a.ctypes.data_as(ctypes.c_void_p)

    fn = _lib().ot_oracle_loss_f32 if dt == np.float32 else _lib().ot_oracle_loss_f64
    rc = fn(ptr(x), ptr(grad), ptr(targets), ptr(T), ptr(U), N, V, max_u,
            int(blank), int(from_log_softmax), int(one_sym_per_frame),
            float(fill), ptr(den), ptr(lp), ptr(alpha), ptr(beta), ptr(sa), ptr(sb))
    if rc != 0:
        raise ValueError(f"oracle rejected its arguments (code {rc})")
    return dict(scores=sa, scores_beta=sb, den=den, lp=lp, alpha=alpha,
                beta=beta, grad=grad)


def band_mask(T, U):
    """Boolean (rows,) mask of the cells the one-symbol-per-frame recursion
    defines: u <= t <= u + (T-1-U) (cpu.cc:295).  Everything else is off-band."""
    out = []
    for t_len, u_len in zip(T, U):
        t = np.arange(t_len)[:, None]
        u = np.arange(u_len + 1)[None, :]
        diff = t_len - 1 - u_len
        out.append(((u <= t) & (t - u <= diff)).reshape(-1))
    return np.concatenate(out)


def brute_force_score(lp_blank, lp_sym, one_sym_per_frame=False):
    """log P(y|x) of ONE utterance by enumerating every alignment.

    ``lp_blank`` and ``lp_sym`` are (T, U+1) arrays of blank / next-symbol
    log-probabilities.  Standard transducer: a path is an interleaving of T-1
    blanks (t -> t+1) and U symbols (u -> u+1) from (0,0) to (T-1,U), then the
    final blank.  One symbol per frame: every one of the first T-1 steps
    advances t and either emits the next symbol (u -> u+1) or a blank.
    Only for tiny lattices (the number of paths is a binomial coefficient).
    """
    lp_blank = np.asarray(lp_blank, np.float64)
    lp_sym = np.asarray(lp_sym, np.float64)
    T, U1 = lp_blank.shape
    U = U1 - 1
    terms = []
    if one_sym_per_frame:
        if U > T - 1:
            return -math.inf
        for sym_steps in itertools.combinations(range(T - 1), U):
            sym_steps = set(sym_steps)
            t = u = 0
            s = 0.0
            for step in range(T - 1):
                if step in sym_steps:
                    s += lp_sym[t, u]
                    u += 1
                else:
                    s += lp_blank[t, u]
                t += 1
            terms.append(s + lp_blank[T - 1, U])
    else:
        for sym_steps in itertools.combinations(range(T - 1 + U), U):
            sym_steps = set(sym_steps)
            t = u = 0
            s = 0.0
            for step in range(T - 1 + U):
                if step in sym_steps:
                    s += lp_sym[t, u]
                    u += 1
                else:
                    s += lp_blank[t, u]
                    t += 1
            terms.append(s + lp_blank[T - 1, U])
    m = max(terms)
    return m + math.log(sum(math.exp(v - m) for v in terms))


def pack_joiner_oracle(encoder_out, decoder_out, T, U):
    """The packing the reference prescribes for the joiner input
    (reference README.md:165-177), in numpy: per utterance the broadcast sum
    ``enc[b,:T_b,None,:] + dec[b,None,:U_b+1,:]`` flattened to rows, then
    concatenated."""
    parts = [(encoder_out[b, :t, None, :] + decoder_out[b, None, :u + 1, :]).reshape(-1, encoder_out.shape[-1])
             for b, (t, u) in enumerate(zip(T, U))]
    return np.concatenate(parts)


def pack_joiner_backward_oracle(grad, T, U, max_t, max_u1):
    """Gradients of :func:`pack_joiner_oracle` w.r.t. its two inputs (float64 sums)."""
    d = grad.shape[-1]
    genc = np.zeros((len(T), max_t, d), np.float64)
    gdec = np.zeros((len(T), max_u1, d), np.float64)
    off = 0
    for b, (t, u) in enumerate(zip(T, U)):
        g = grad[off:off + t * (u + 1)].reshape(t, u + 1, d).astype(np.float64)
        genc[b, :t] = g.sum(1)
        gdec[b, :u + 1] = g.sum(0)
        off += t * (u + 1)
    return genc, gdec


def pack_padded_oracle(padded, T, U):
    """Padded (N, maxT, maxU+1, D) -> packed rows, as the reference's tests slice it
    (python/tests/test_compute_transducer_loss.py:36-56)."""
    return np.concatenate([padded[b, :t, :u + 1, :].reshape(-1, padded.shape[-1])
                           for b, (t, u) in enumerate(zip(T, U))])


def _import_so(name, path):
    loader = importlib.machinery.ExtensionFileLoader(name, path)
    spec = importlib.util.spec_from_file_location(name, path, loader=loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    return mod


def load_ref():
    """Returns ``(reference_extension, stage_shim)`` from ``oracle/_ref`` or
    ``None`` when the reference build is not present.  Needs torch."""
    if "mods" not in _REF:
        a = os.path.join(HERE, "_ref", "_optimized_transducer", "_optimized_transducer.so")
        b = os.path.join(HERE, "_ref", "_ot_ref_stages", "_ot_ref_stages.so")
        if os.path.isfile(a) and os.path.isfile(b):
            import torch  # noqa: F401  (the extensions link against libtorch)
            _REF["mods"] = (_import_so("_optimized_transducer", a),
                            _import_so("_ot_ref_stages", b))
        else:
            _REF["mods"] = None
    return _REF["mods"]


def load_ref_python(cuda=False):
    """The reference's own Python layer (``transducer_loss.py`` as installed under
    ``oracle/_ref/python`` by ``build_ref.py``) bound to the reference's own
    extension, or None when either is missing.  ``cuda=True`` binds it to the
    build that includes the reference's CUDA kernels
    (``oracle/_ref/_optimized_transducer_cuda``, ``build_ref.build_cuda``) instead
    of the CPU-only one.  The module does ``import _optimized_transducer`` at
    import time; that name is bound to the reference build for the duration of
    the import only."""
    key = "py_cuda" if cuda else "py"
    if key not in _REF:
        path = os.path.join(HERE, "_ref", "python", "transducer_loss.py")
        if cuda:
            so = os.path.join(HERE, "_ref", "_optimized_transducer_cuda", "_optimized_transducer.so")
            ext = None
            if os.path.isfile(so):
                import torch  # noqa: F401
                ext = _import_so("_optimized_transducer", so)
        else:
            mods = load_ref()
            ext = None if mods is None else mods[0]
        if ext is None or not os.path.isfile(path):
            _REF[key] = None
        else:
            import sys
            saved = sys.modules.get("_optimized_transducer")
            sys.modules["_optimized_transducer"] = ext
            try:
                spec = importlib.util.spec_from_file_location("_ot_reference_transducer_loss_" + key, path)
                mod = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(mod)
            finally:
                if saved is None:
                    sys.modules.pop("_optimized_transducer", None)
                else:
                    sys.modules["_optimized_transducer"] = saved
            _REF[key] = mod
    return _REF[key]


def ref_loss(x, targets, T, U, blank, from_log_softmax=False,
             one_sym_per_frame=False, want_grad=True):
    """Calls the reference's own ``compute_transducer_loss`` (float32, CPU).

    Returns ``(scores, grad)`` as numpy arrays; ``grad`` is None unless
    ``want_grad``.  ``x`` is not modified (a copy is handed to the reference,
    which overwrites its input when ``from_log_softmax`` is False,
    cpu.cc:814)."""
    import torch

    ext, _ = load_ref()
    lx = torch.from_numpy(np.array(x, np.float32, copy=True)).requires_grad_(want_grad)
    scores, grad = ext.compute_transducer_loss(
        logits=lx, targets=torch.from_numpy(np.ascontiguousarray(targets, np.int32)),
        logit_lengths=torch.from_numpy(np.ascontiguousarray(T, np.int32)),
        target_lengths=torch.from_numpy(np.ascontiguousarray(U, np.int32)),
        blank=int(blank), from_log_softmax=bool(from_log_softmax),
        one_sym_per_frame=bool(one_sym_per_frame))
    return scores.detach().numpy(), (None if grad is None else grad.detach().numpy())


def ref_stages(x, targets, T, U, blank, from_log_softmax=False,
               one_sym_per_frame=False):
    """log-probs, alpha, beta and the two score vectors from the reference's
    file-static stage functions (through ``ref_stage_shim.cc``)."""
    import torch

    _, shim = load_ref()
    tt = torch.from_numpy(np.ascontiguousarray(T, np.int32))
    tu = torch.from_numpy(np.ascontiguousarray(U, np.int32))
    lp = shim.log_probs(torch.from_numpy(np.ascontiguousarray(x, np.float32)),
                        torch.from_numpy(np.ascontiguousarray(targets, np.int32)),
                        tt, tu, int(blank), bool(from_log_softmax))
    alpha, sa = shim.alpha(lp, tt, tu, bool(one_sym_per_frame))
    beta, sb = shim.beta(lp, tt, tu, bool(one_sym_per_frame))
    return dict(lp=lp.numpy(), alpha=alpha.numpy(), beta=beta.numpy(),
                scores=sa.numpy(), scores_beta=sb.numpy())
