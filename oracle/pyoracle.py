"""ctypes access to the CPU oracle (oracle/sumcheck_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's
CPU-baseline legs, never by the product package.
"""
import ctypes as C
import os
import subprocess

import numpy as np

P = 2130706433
_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

u32p = C.POINTER(C.c_uint32)


def build():
    """Compile liboracle.so next to its source (gcc, OpenMP)."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "liboracle.so"])


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        src = os.path.join(_HERE, "sumcheck_oracle.c")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
            build()
        _LIB = C.CDLL(path)
        _LIB.orc_tr_new.restype = C.c_void_p
        _LIB.orc_tr_encode.restype = C.c_uint64
        _LIB.orc_tr_sent_bytes.restype = C.c_uint64
        _LIB.orc_fpow.restype = C.c_uint32
    return _LIB


def _u32(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.uint32))


def _ptr(a):
    return a.ctypes.data_as(u32p)


def _strs(names):
    arr = (C.c_char_p * max(len(names), 1))()
    for i, s in enumerate(names):
        arr[i] = s.encode()
    return arr


def ext_op(name, D, a, b=None):
    out = np.zeros(D, dtype=np.uint32)
    a = _u32(a)
    if b is None:
        getattr(lib(), name)(C.c_int(D), _ptr(a), _ptr(out))
    else:
        b = _u32(b)
        getattr(lib(), name)(C.c_int(D), _ptr(a), _ptr(b), _ptr(out))
    return out.tolist()


def ext_mul(D, a, b): return ext_op("orc_ext_mul", D, a, b)
def ext_add(D, a, b): return ext_op("orc_ext_add", D, a, b)
def ext_sub(D, a, b): return ext_op("orc_ext_sub", D, a, b)
def ext_eq1(D, a, b): return ext_op("orc_ext_eq1", D, a, b)
def ext_inv(D, a): return ext_op("orc_ext_inv", D, a)
def fpow(a, e): return int(lib().orc_fpow(C.c_uint32(a), C.c_uint64(e)))


def eq_table(D, r):
    r = _u32(r).reshape(-1, D) if len(r) else np.zeros((0, D), dtype=np.uint32)
    out = np.zeros((1 << len(r), D), dtype=np.uint32)
    lib().orc_eq_table(C.c_int(D), C.c_int(len(r)), _ptr(r), _ptr(out))
    return out


def lagrange(D, values, x):
    values = _u32(values).reshape(-1, D)
    x = _u32(x)
    out = np.zeros(D, dtype=np.uint32)
    lib().orc_lagrange(C.c_int(D), C.c_int(len(values)), _ptr(values), _ptr(x), _ptr(out))
    return out.tolist()


def mle_eval(D, values, r):
    values = _u32(values)
    stride = 1 if values.ndim == 1 else D
    r = _u32(r).reshape(-1, D) if len(r) else np.zeros((0, D), dtype=np.uint32)
    out = np.zeros(D, dtype=np.uint32)
    lib().orc_mle_eval(C.c_int(D), C.c_int(len(r)), _ptr(values), C.c_int(stride), _ptr(r), _ptr(out))
    return out.tolist()


def b3s(chunks, n):
    bufs = [C.create_string_buffer(c, len(c)) for c in chunks]
    ptrs = (C.c_void_p * max(len(chunks), 1))(*[C.addressof(b) for b in bufs])
    lens = (C.c_uint64 * max(len(chunks), 1))(*[len(c) for c in chunks])
    out = C.create_string_buffer(n)
    lib().orc_b3s(ptrs, lens, C.c_int(len(chunks)), out, C.c_uint64(n))
    return out.raw


def expand(statement, variables, cap=256):
    """EXPAND's terms as (indices into VARIABLES, coefficient), in graded order."""
    degs = (C.c_int * cap)()
    idx = (C.c_int * (cap * 24))()
    coeffs = (C.c_uint32 * cap)()
    n = lib().orc_expand(statement.encode(), C.c_int(len(variables)), _strs(variables), C.c_int(cap), degs, idx, coeffs)
    if n < 0:
        raise ValueError("cannot expand %r" % statement)
    return [([idx[24 * i + k] for k in range(degs[i])], int(coeffs[i])) for i in range(n)]


def statement_degree(statement, tables, constants=()):
    d = lib().orc_statement_degree(statement.encode(), C.c_int(len(tables)), _strs(list(tables)),
                                   C.c_int(len(constants)), _strs(list(constants)))
    if d < 0:
        raise ValueError("bad statement %r" % statement)
    return d


class Transcript:
    """The Fiat-Shamir transcript (reference src/transcript.lisp), prover side."""

    def __init__(self, label, degree):
        if isinstance(label, str):
            label = label.encode()
        self.label = label
        self.degree = degree
        self._h = C.c_void_p(lib().orc_tr_new(label, C.c_int(len(label)), C.c_int(degree)))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_tr_free(self._h)
            self._h = None

    def absorb(self, data):
        lib().orc_tr_absorb(self._h, bytes(data), C.c_uint64(len(data)))

    def send(self, values):
        values = _u32(values)
        rows, cols = values.shape
        lib().orc_tr_send(self._h, _ptr(values), C.c_int(rows), C.c_int(cols))

    def challenge_base(self, k):
        out = np.zeros(k, dtype=np.uint32)
        lib().orc_tr_challenge_base(self._h, C.c_int(k), _ptr(out))
        return out.tolist()

    def challenge(self, degree=None):
        return self.challenge_base(degree or self.degree)

    def challenge_bits(self, nbits, k):
        out = (C.c_uint64 * k)()
        lib().orc_tr_challenge_bits(self._h, C.c_int(nbits), C.c_int(k), out)
        return list(out)

    def digest(self, n=32):
        out = C.create_string_buffer(n)
        lib().orc_tr_digest(self._h, out, C.c_int(n))
        return out.raw

    def messages(self):
        out = []
        for i in range(lib().orc_tr_nmessages(self._h)):
            dims = (C.c_uint64 * 2)()
            lib().orc_tr_message(self._h, C.c_int(i), dims, None)
            vals = np.zeros((dims[0], dims[1]), dtype=np.uint32)
            lib().orc_tr_message(self._h, C.c_int(i), dims, _ptr(vals))
            out.append(vals)
        return out

    def sent_bytes(self):
        return int(lib().orc_tr_sent_bytes(self._h))

    def proof(self, magic=b"EXACTPF1"):
        need = lib().orc_tr_encode(self._h, magic, None, C.c_uint64(0))
        buf = C.create_string_buffer(need)
        lib().orc_tr_encode(self._h, magic, buf, C.c_uint64(need))
        return buf.raw


def _tables(tables, D, entries):
    names, arrays, strides = [], [], []
    for name, values in tables:
        a = _u32(values)
        stride = 1 if a.ndim == 1 else a.shape[1]
        if stride not in (1, D) or a.shape[0] != entries:
            raise ValueError("table %s: shape %s" % (name, a.shape))
        names.append(name); arrays.append(a); strides.append(stride)
    ptrs = (u32p * max(len(arrays), 1))(*[_ptr(a) for a in arrays])
    return names, arrays, ptrs, (C.c_int * max(len(arrays), 1))(*strides)


def _constants(constants, D):
    names = [c[0] for c in constants]
    vals = _u32([c[1] for c in constants]).reshape(-1, D) if constants else np.zeros((1, D), dtype=np.uint32)
    return names, vals


def prove(tr, n, statement, tables, eq=None, constants=(), label="sc", block_weights=None, degree=None,
          threads=1):
    """The reference's (prove tr n statement tables :eq :constants :label :block-weights :degree).

    tables: list of (name, array) with arrays of shape (K 2^n,) for base tables or (K 2^n, D).
    Returns (challenges [n][D], finals {name: [D]}, folded {name: [K][D]}).
    """
    D = tr.degree
    K = 0 if block_weights is None else len(block_weights)
    blocks = max(K, 1)
    names, arrays, ptrs, strides = _tables(tables, D, blocks << n)
    cnames, cvals = _constants(list(constants), D)
    eqa = _u32(eq).reshape(-1, D) if eq is not None else None
    bwa = _u32(block_weights).reshape(-1, D) if K else None
    ch = np.zeros((max(n, 1), D), dtype=np.uint32)
    fin = np.zeros((max(len(names), 1), D), dtype=np.uint32)
    fol = np.zeros((max(len(names), 1), blocks, D), dtype=np.uint32)
    rc = lib().orc_prove(tr._h, C.c_int(n), statement.encode(), C.c_int(len(names)), _strs(names), ptrs, strides,
                         _ptr(eqa) if eqa is not None else None, C.c_int(len(cnames)), _strs(cnames), _ptr(cvals),
                         label.encode(), C.c_int(K), _ptr(bwa) if K else None,
                         C.c_int(-1 if degree is None else degree), C.c_int(threads), _ptr(ch), _ptr(fin), _ptr(fol))
    if rc:
        raise ValueError("oracle prove failed: %d" % rc)
    return (ch[:n].tolist(), {nm: fin[i].tolist() for i, nm in enumerate(names)},
            {nm: fol[i].tolist() for i, nm in enumerate(names)})


def hypercube_sum(D, n, statement, tables, eq=None, constants=()):
    names, arrays, ptrs, strides = _tables(tables, D, 1 << n)
    cnames, cvals = _constants(list(constants), D)
    eqa = _u32(eq).reshape(-1, D) if eq is not None else None
    out = np.zeros(D, dtype=np.uint32)
    rc = lib().orc_hypercube_sum(C.c_int(D), C.c_int(n), statement.encode(), C.c_int(len(names)), _strs(names), ptrs,
                                 strides, _ptr(eqa) if eqa is not None else None, C.c_int(len(cnames)),
                                 _strs(cnames), _ptr(cvals), _ptr(out))
    if rc:
        raise ValueError("oracle hypercube_sum failed: %d" % rc)
    return out.tolist()


def verify(tr_label, D, n, degree, claim, messages, eq=None, blocks=1, label="sc"):
    """Replay a proof (reference verify); returns (challenges, reduced claim)."""
    if isinstance(tr_label, str):
        tr_label = tr_label.encode()
    msgs = _u32(np.concatenate([_u32(m).reshape(-1) for m in messages])) if n else np.zeros(1, dtype=np.uint32)
    eqa = _u32(eq).reshape(-1, D) if eq is not None else None
    claim = _u32(claim)
    ch = np.zeros((max(n, 1), D), dtype=np.uint32)
    red = np.zeros(D, dtype=np.uint32)
    lib().orc_verify(tr_label, C.c_int(len(tr_label)), C.c_int(D), C.c_int(n), C.c_int(degree), _ptr(claim),
                     _ptr(eqa) if eqa is not None else None, C.c_int(blocks), label.encode(), _ptr(msgs), _ptr(ch),
                     _ptr(red))
    return ch[:n].tolist(), red.tolist()


def check_final(D, statement, finals, reduced, constants=()):
    names = [f[0] for f in finals]
    vals = _u32([f[1] for f in finals]).reshape(-1, D) if finals else np.zeros((1, D), dtype=np.uint32)
    cnames, cvals = _constants(list(constants), D)
    red = _u32(reduced)
    return lib().orc_check_final(C.c_int(D), statement.encode(), C.c_int(len(names)), _strs(names), _ptr(vals),
                                 C.c_int(len(cnames)), _strs(cnames), _ptr(cvals), _ptr(red)) == 1


def generate(seed, table_id, first, count, stride, nonzero=False):
    out = np.zeros(count * stride, dtype=np.uint32)
    lib().orc_generate(C.c_uint64(seed), C.c_int(table_id), C.c_uint64(first), C.c_uint64(count), C.c_int(stride),
                       C.c_int(1 if nonzero else 0), _ptr(out))
    return out if stride == 1 else out.reshape(count, stride)


def max_threads():
    return int(lib().orc_max_threads())
