"""sable_b200 -- the sumcheck prover of Exacta (drvova/Sable) on a B200.

This package is the thin Python face of libsumcheck_b200.so (CUDA, sm_100a; built by
``python -m sable_b200.build``).  It mirrors the reference's operator for this path,

    (exacta.sumcheck:prove tr n statement tables &key eq constants label block-weights degree)

(reference src/sumcheck.lisp:512-571) with the same argument meaning and the same results: the
round challenges, the finals and the folded tables, and a transcript that ends in the same state
with the same recorded messages, so the proof bytes are the reference's.

There is no CPU path: without the built library, or without a CUDA device, the calls raise.
"""
import ctypes as C
import os

import numpy as np

P = 2130706433                      # the KoalaBear prime 2^31 - 2^24 + 1 (reference src/field.lisp:31)
MAGIC = b"EXACTPF1"                 # reference src/proofio.lisp:18

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY = os.environ.get("SABLE_B200_LIBRARY", os.path.join(_HERE, "libsumcheck_b200.so"))
_lib = None
_u32p = C.POINTER(C.c_uint32)

SYMBOLS = [
    "sc_create", "sc_destroy", "sc_set_memory_budget", "sc_strerror", "sc_last_error", "sc_set_statement",
    "sc_upload_table", "sc_generate_table", "sc_download_table", "sc_begin", "sc_round", "sc_challenge", "sc_finish",
    "sc_enable_timing", "sc_round_stats", "sc_launch_count", "sc_timer_start", "sc_timer_stop", "sc_fetch_table", "sc_comm_unique_id", "sc_comm_init", "sc_comm_info", "sc_round_sums_static",
    "sc_transcript_new", "sc_transcript_free", "sc_transcript_absorb", "sc_transcript_send",
    "sc_transcript_challenge_base", "sc_transcript_challenge_bits", "sc_transcript_digest",
    "sc_transcript_message_count", "sc_transcript_message", "sc_transcript_sent_bytes", "sc_transcript_encode",
    "sc_lower_statement", "sc_prove", "sc_borrow_table", "sc_transcript_degree", "sc_gkr_prove_upper", "sc_reserve", "sc_workspace", "sc_child", "sc_attach_transcript", "sc_transcript_state",
    "sc_transcript_device_round", "sc_attach_transcript_state", "sc_set_device_transcript", "sc_domain_statement", "sc_prove_domain",
]


class SumcheckError(RuntimeError):
    """A call into the library failed; ``code`` is its SC_E* value."""

    def __init__(self, code, message):
        super().__init__("%s (code %d)" % (message, code))
        self.code = code


class InvalidParameter(SumcheckError, ValueError):
    """The reference's INVALID-PARAMETER (src/conditions.lisp:94-122)."""


def library():
    """The loaded shared library; raises if it was never built (there is no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIBRARY):
            raise ImportError("%s is missing: build it with `python -m sable_b200.build`" % LIBRARY)
        lib = C.CDLL(LIBRARY)
        lib.sc_strerror.restype = C.c_char_p
        lib.sc_last_error.restype = C.c_char_p
        lib.sc_last_error.argtypes = [C.c_void_p]
        lib.sc_transcript_new.restype = C.c_void_p
        lib.sc_transcript_new.argtypes = [C.c_char_p, C.c_size_t, C.c_int]
        lib.sc_transcript_free.argtypes = [C.c_void_p]
        lib.sc_transcript_sent_bytes.restype = C.c_uint64
        lib.sc_transcript_sent_bytes.argtypes = [C.c_void_p]
        lib.sc_transcript_encode.restype = C.c_uint64
        lib.sc_launch_count.restype = C.c_uint64
        lib.sc_launch_count.argtypes = [C.c_void_p]
        _lib = lib
    return _lib


def _check(code, ctx=None):
    if code == 0:
        return
    lib = library()
    text = lib.sc_strerror(code).decode()
    if ctx is not None:
        detail = lib.sc_last_error(ctx).decode()
        if detail:
            text = "%s: %s" % (text, detail)
    raise (InvalidParameter if code in (-1, -7) else SumcheckError)(code, text)


def _u32(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.uint32))


def _ptr(a):
    return a.ctypes.data_as(_u32p)


def _strs(names):
    arr = (C.c_char_p * max(len(names), 1))()
    for i, s in enumerate(names):
        arr[i] = s.encode()
    return arr


class Transcript:
    """The Fiat-Shamir transcript, prover side (reference MAKE-TRANSCRIPT, src/transcript.lisp:75-84)."""

    def __init__(self, label, degree):
        if isinstance(label, str):
            label = label.encode()
        self.degree = degree
        self._h = library().sc_transcript_new(label, len(label), degree)
        if not self._h:
            raise InvalidParameter(-1, "extension degree %r: expected 4 or 8" % (degree,))

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.sc_transcript_free(self._h)
            self._h = None

    def absorb(self, data):
        data = bytes(data)
        _check(library().sc_transcript_absorb(C.c_void_p(self._h), data, C.c_uint64(len(data))))

    def send(self, values):
        values = _u32(values)
        rows, cols = values.shape
        _check(library().sc_transcript_send(C.c_void_p(self._h), _ptr(values), rows, cols))

    def challenge_base(self, k):
        out = np.zeros(max(k, 1), dtype=np.uint32)
        _check(library().sc_transcript_challenge_base(C.c_void_p(self._h), k, _ptr(out)))
        return out[:k].tolist()

    def challenge(self, degree=None):
        return self.challenge_base(degree or self.degree)

    def challenge_bits(self, nbits, k):
        out = (C.c_uint64 * max(k, 1))()
        _check(library().sc_transcript_challenge_bits(C.c_void_p(self._h), nbits, k, out))
        return list(out)[:k]

    def digest(self, n=32):
        out = C.create_string_buffer(n)
        _check(library().sc_transcript_digest(C.c_void_p(self._h), out, C.c_size_t(n)))
        return out.raw

    @property
    def messages(self):
        """The field arrays sent so far (reference TRANSCRIPT-MESSAGES)."""
        lib = library()
        out = []
        for i in range(lib.sc_transcript_message_count(C.c_void_p(self._h))):
            dims = (C.c_uint64 * 2)()
            lib.sc_transcript_message(C.c_void_p(self._h), i, dims, None)
            vals = np.zeros((dims[0], dims[1]), dtype=np.uint32)
            lib.sc_transcript_message(C.c_void_p(self._h), i, dims, _ptr(vals))
            out.append(vals)
        return out

    @property
    def sent_bytes(self):
        return int(library().sc_transcript_sent_bytes(C.c_void_p(self._h)))

    def proof(self, magic=MAGIC):
        """The proof bytes of the recorded messages (reference ENCODE-PROOF, src/proofio.lisp:44-49)."""
        lib = library()
        need = lib.sc_transcript_encode(C.c_void_p(self._h), magic, None, C.c_uint64(0))
        buf = C.create_string_buffer(need)
        lib.sc_transcript_encode(C.c_void_p(self._h), magic, buf, C.c_uint64(need))
        return buf.raw


def lower_statement(statement, degree_d, tables, constants=()):
    """The statement as a term table: (degree, [(coefficient words, table indices)...]).

    ``tables`` are the table names in slot order; ``constants`` pairs (name, D words).
    """
    lib = library()
    D = degree_d
    cnames = [c[0] for c in constants]
    cvals = _u32([c[1] for c in constants]).reshape(-1, D) if constants else np.zeros((1, D), dtype=np.uint32)
    deg, nterms = C.c_int(0), C.c_int(0)
    coeffs = np.zeros((16, D), dtype=np.uint32)
    ptr = np.zeros(17, dtype=np.int32)
    idx = np.zeros(16 * 8, dtype=np.int32)
    _check(lib.sc_lower_statement(statement.encode(), D, len(tables), _strs(list(tables)), len(cnames), _strs(cnames),
                                  _ptr(cvals), C.byref(deg), C.byref(nterms), _ptr(coeffs),
                                  ptr.ctypes.data_as(C.POINTER(C.c_int32)), idx.ctypes.data_as(C.POINTER(C.c_int32))))
    terms = [(coeffs[t].tolist(), idx[ptr[t]:ptr[t + 1]].tolist()) for t in range(nterms.value)]
    return deg.value, terms


class RoundStat(C.Structure):
    _fields_ = [("kernel_ms", C.c_float), ("bytes", C.c_uint64), ("pairs", C.c_uint64)]


class Prover:
    """A device context: it owns the tables and every buffer of a proof on one GPU."""

    def __init__(self, device=0):
        self._h = C.c_void_p()
        code = library().sc_create(device, C.byref(self._h))
        if code:
            self._h = None
            _check(code)

    def close(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.sc_destroy(self._h)
        self._h = None

    __del__ = close

    def _call(self, name, *args):
        _check(getattr(library(), name)(self._h, *args), self._h)

    # -- the device layer, one method per C function
    def set_memory_budget(self, nbytes):
        self._call("sc_set_memory_budget", C.c_uint64(nbytes))

    def set_statement(self, D, points, ntables, terms):
        coeffs = _u32([t[0] for t in terms]).reshape(-1, D) if terms else np.zeros((1, D), dtype=np.uint32)
        ptr = np.zeros(len(terms) + 1, dtype=np.int32)
        idx = []
        for i, (_, tabs) in enumerate(terms):
            idx.extend(tabs)
            ptr[i + 1] = len(idx)
        idx = np.asarray(idx + [0], dtype=np.int32)
        self._call("sc_set_statement", D, points, ntables, len(terms), _ptr(coeffs),
                   ptr.ctypes.data_as(C.POINTER(C.c_int32)), idx.ctypes.data_as(C.POINTER(C.c_int32)))
        self._D, self._points = D, points

    def upload_table(self, slot, values):
        a = _u32(values)
        stride = 1 if a.ndim == 1 else a.shape[1]
        self._call("sc_upload_table", slot, _ptr(a), C.c_uint64(a.shape[0]), stride)

    def upload_pointer(self, slot, address, entries, stride):
        """Upload from raw host memory (for example pinned memory) at ``address``."""
        self._call("sc_upload_table", slot, C.cast(C.c_void_p(address), _u32p), C.c_uint64(entries), stride)

    def borrow_table(self, slot, address, entries, stride):
        """Table ``slot`` is the caller's device memory at ``address`` (canonical words); nothing is copied."""
        self._call("sc_borrow_table", slot, C.cast(C.c_void_p(address), _u32p), C.c_uint64(entries), stride)

    def generate_table(self, slot, seed, table_id, entries, stride, first=0, nonzero=False):
        self._call("sc_generate_table", slot, C.c_uint64(seed), table_id, C.c_uint64(first), C.c_uint64(entries), stride,
                   1 if nonzero else 0)

    def download_table(self, slot, D, cap=None):
        n = C.c_uint64(0)
        self._call("sc_download_table", slot, None, C.c_uint64(0), C.byref(n))
        count = n.value if cap is None else min(n.value, cap)
        out = np.zeros((count, D), dtype=np.uint32)
        self._call("sc_download_table", slot, _ptr(out), C.c_uint64(count), C.byref(n))
        return out

    def begin(self, n, eq=None, block_weights=None):
        eqa = _u32(eq).reshape(-1, self._D) if eq is not None else None
        if eqa is not None and len(eqa) < n:
            raise InvalidParameter(-1, "eq has %d elements: expected at least %d" % (len(eqa), n))
        bwa = _u32(block_weights).reshape(-1, self._D) if block_weights is not None else None
        self._call("sc_begin", n, _ptr(eqa) if eqa is not None else None, len(bwa) if bwa is not None else 1,
                   _ptr(bwa) if bwa is not None else None)

    def round(self):
        out = np.zeros((self._points, self._D), dtype=np.uint32)
        self._call("sc_round", _ptr(out))
        return out

    def challenge(self, r):
        r = _u32(r)
        self._call("sc_challenge", _ptr(r))

    def finish(self, ntables, K=1):
        out = np.zeros((ntables, K, self._D), dtype=np.uint32)
        self._call("sc_finish", _ptr(out))
        return out

    def enable_timing(self, on=True):
        self._call("sc_enable_timing", 1 if on else 0)

    def round_stats(self):
        count = C.c_int(0)
        stats = (RoundStat * 64)()
        self._call("sc_round_stats", stats, 64, C.byref(count))
        return [(s.kernel_ms, s.bytes, s.pairs) for s in stats[:count.value]]

    def timer_start(self):
        self._call("sc_timer_start")

    def timer_stop(self):
        ms = C.c_float(0)
        self._call("sc_timer_stop", C.byref(ms))
        return ms.value

    def fetch_pointer(self, slot, address, words):
        """Copy the caller's words of table ``slot`` from the device to host memory at ``address``."""
        self._call("sc_fetch_table", slot, C.cast(C.c_void_p(address), _u32p), C.c_uint64(words))

    @property
    def launches(self):
        return int(library().sc_launch_count(self._h))

    def set_device_transcript(self, on=True):
        """Carry the transcript on the device: every round of a proof is enqueued at once (sc_set_device_transcript)."""
        self._call("sc_set_device_transcript", 1 if on else 0)

    def attach_transcript(self, tr):
        """The host transcript of the proofs that follow (or None); needed by the device transcript."""
        self._call("sc_attach_transcript", C.c_void_p(tr._h) if tr is not None else None)

    def comm_init(self, unique_id, rank, world):
        self._call("sc_comm_init", unique_id, rank, world)

    @property
    def world(self):
        """Ranks of the communicator (1 without one); with several, each rank's tables are its slice."""
        w = C.c_int(1)
        self._call("sc_comm_info", None, C.byref(w))
        return w.value


def round_sums_static(D, points, tables_dev, strides, entries, terms, sums_dev, stream=0):
    """Round-0 sums without eq weights over device-resident tables, with no allocation (sc_round_sums_static).

    For callers that cannot allocate device memory where they run.  ``tables_dev`` and ``sums_dev``
    are device addresses (integers) the caller owns; ``terms`` is the term table as for
    ``Prover.set_statement``.  The launch is asynchronous on ``stream``; calls share one fixed
    scratch array in the library, so calls that overlap on the GPU race.  At most 2^28 entries.
    """
    coeffs = _u32([t[0] for t in terms]).reshape(-1, D) if terms else np.zeros((1, D), dtype=np.uint32)
    ptr = np.zeros(len(terms) + 1, dtype=np.int32)
    idx = []
    for i, (_, tabs) in enumerate(terms):
        idx.extend(tabs)
        ptr[i + 1] = len(idx)
    idx = np.asarray(idx + [0], dtype=np.int32)
    tabs = (_u32p * max(len(tables_dev), 1))(*[C.cast(C.c_void_p(a), _u32p) for a in tables_dev])
    message = C.create_string_buffer(512)
    code = library().sc_round_sums_static(D, points, len(tables_dev), tabs, (C.c_int * max(len(strides), 1))(*strides),
                                          C.c_uint64(entries), len(terms), _ptr(coeffs), ptr.ctypes.data_as(C.POINTER(C.c_int32)),
                                          idx.ctypes.data_as(C.POINTER(C.c_int32)), C.cast(C.c_void_p(sums_dev), _u32p),
                                          C.c_void_p(stream), message, C.c_size_t(512))
    if code:
        text = "%s: %s" % (library().sc_strerror(code).decode(), message.value.decode())
        raise (InvalidParameter if code in (-1, -7) else SumcheckError)(code, text)


def comm_unique_id():
    """A fresh 128-byte NCCL id (made on rank 0 and handed to every rank)."""
    buf = C.create_string_buffer(128)
    _check(library().sc_comm_unique_id(buf))
    return buf.raw


class DeviceTable:
    """A table already on the device in the slot it is listed at (uploaded or generated earlier)."""

    def __init__(self, stride):
        self.stride = stride


_default_prover = None


def default_prover():
    global _default_prover
    if _default_prover is None:
        _default_prover = Prover(0)
    return _default_prover


def prove(tr, n, statement, tables, eq=None, constants=(), label="sc", block_weights=None, degree=None, prover=None):
    """The reference's PROVE (src/sumcheck.lisp:512-571) with its argument meaning.

    tr             a prover Transcript; its extension degree D is the proof's
    n              number of variables (rounds)
    statement      the form as text, e.g. "(+ (* alpha t0 t1) (* 3 t1))"
    tables         pairs (name, values): K 2^n base elements (shape (N,)) or extension elements
                   (shape (N, D)); or a DeviceTable for a table already in that slot
    eq             at least n extension elements, or None (weights 1)
    constants      pairs (name, D words) for the statement's variables that are not tables
    block_weights  K extension elements: tables hold K blocks of 2^n entries, block-major
    degree         the degree the header states (default: the statement's degree in the tables)

    Returns (challenges, finals, folded): n challenges of D words; {name: D words} at block 0;
    {name: K x D words}.
    """
    prover = prover or default_prover()
    lib = library()
    D = tr.degree
    K = 1 if block_weights is None else len(block_weights)
    names, arrays, strides = [], [], []
    for name, values in tables:
        names.append(name)
        if isinstance(values, DeviceTable):
            arrays.append(None)
            strides.append(values.stride)
            continue
        a = _u32(values)
        stride = 1 if a.ndim == 1 else a.shape[1]
        if a.ndim > 2 or stride not in (1, D) or a.shape[0] != (K << n) // prover.world:
            raise InvalidParameter(-1, "table %s of shape %s: expected %d base elements or extension elements of degree %d"
                                   % (name, a.shape, (K << n) // prover.world, D))
        arrays.append(a)
        strides.append(stride)
    ptrs = (_u32p * max(len(names), 1))(*[_ptr(a) if a is not None else None for a in arrays])
    cnames = [c[0] for c in constants]
    cvals = _u32([c[1] for c in constants]).reshape(-1, D) if cnames else np.zeros((1, D), dtype=np.uint32)
    eqa = None
    if eq is not None:
        eqa = _u32(eq).reshape(-1, D)
        if len(eqa) < n:
            raise InvalidParameter(-1, "eq has %d elements: expected at least %d" % (len(eqa), n))
    bwa = _u32(block_weights).reshape(-1, D) if block_weights is not None else None
    ch = np.zeros((max(n, 1), D), dtype=np.uint32)
    fin = np.zeros((max(len(names), 1), D), dtype=np.uint32)
    fol = np.zeros((max(len(names), 1), K, D), dtype=np.uint32)
    code = lib.sc_prove(prover._h, C.c_void_p(tr._h), n, statement.encode(), len(names), _strs(names), ptrs,
                        (C.c_int * max(len(names), 1))(*strides), _ptr(eqa) if eqa is not None else None, len(cnames),
                        _strs(cnames), _ptr(cvals), label.encode(), K, _ptr(bwa) if bwa is not None else None,
                        -1 if degree is None else degree, _ptr(ch), _ptr(fin), _ptr(fol))
    _check(code, prover._h)
    return (ch[:n].tolist(), {nm: fin[i].tolist() for i, nm in enumerate(names)},
            {nm: fol[i].tolist() for i, nm in enumerate(names)})


_gkr_provers = []


def gkr_prove_upper(tr, n, k, leaves, label="gkr", provers=None):
    """The reference's (prove-upper tr n k leaves :label label), src/gkr.lisp:215-272.

    leaves: a list, one (p, q) per lookup, of arrays of shape (k 2^n, D), block-major (numpy arrays,
    or CUDA tensors of 32-bit words, which are read where they lie).  provers: one
    Prover per lookup (made and kept when not given).  Returns (ri, rb, cp, cq) as lists of D-word lists.
    """
    D = tr.degree
    lookups = len(leaves)
    if provers is None:
        while len(_gkr_provers) < lookups:
            _gkr_provers.append(Prover(0))
        provers = _gkr_provers[:lookups]
    on_device = all(hasattr(a, "data_ptr") for pq in leaves for a in pq)   # device tensors (uint32/int32, contiguous): read in place
    if on_device:
        ps, qs = [p for p, _ in leaves], [q for _, q in leaves]
        for a in ps + qs:
            if not a.is_cuda or not a.is_contiguous() or a.element_size() != 4 or a.numel() != (k << n) * D:
                raise InvalidParameter(-1, "device leaves: expected contiguous 32-bit tensors of %d words" % ((k << n) * D))
        address = lambda a: C.cast(C.c_void_p(a.data_ptr()), _u32p)
    else:
        ps = [_u32(p).reshape(-1, D) for p, _ in leaves]
        qs = [_u32(q).reshape(-1, D) for _, q in leaves]
        for a in ps + qs:
            if a.shape[0] != k << n:
                raise InvalidParameter(-1, "leaves of %d entries: expected %d" % (a.shape[0], k << n))
        address = _ptr
    lk = (k - 1).bit_length()
    ri = np.zeros((max(n - 1, 1), D), dtype=np.uint32)
    rb = np.zeros((max(lk, 1), D), dtype=np.uint32)
    cp = np.zeros((lookups, D), dtype=np.uint32)
    cq = np.zeros((lookups, D), dtype=np.uint32)
    ctxs = (C.c_void_p * lookups)(*[p._h.value for p in provers])
    pp = (_u32p * lookups)(*[address(a) for a in ps])
    qp = (_u32p * lookups)(*[address(a) for a in qs])
    rc = library().sc_gkr_prove_upper(ctxs, lookups, C.c_void_p(tr._h), n, k, pp, qp, 1 if on_device else 0, label.encode(), _ptr(ri), _ptr(rb), _ptr(cp), _ptr(cq))
    if rc:
        for p in provers:      # the context that failed holds the message
            detail = library().sc_last_error(p._h).decode()
            if detail:
                _check(rc, p._h)
        _check(rc)
    return ri[:n - 1].tolist(), rb[:lk].tolist(), cp.tolist(), cq.tolist()


# ------------------------------------------------------------------ domains (reference src/domain.lisp)

class _DomainColumn(C.Structure):
    _fields_ = [("name", C.c_char_p), ("kind", C.c_int), ("c", C.c_int), ("shared", C.c_int), ("data", _u32p)]


class _DomainLookup(C.Structure):
    _fields_ = [("tag", C.c_char_p), ("nvalues", C.c_int), ("values", C.POINTER(C.c_char_p)), ("num", C.c_char_p)]


class _Domain(C.Structure):
    _fields_ = [("name", C.c_char_p), ("n", C.c_int), ("blocks", C.c_int), ("merge", C.c_int),
                ("ncolumns", C.c_int), ("columns", C.POINTER(_DomainColumn)),
                ("nconstraints", C.c_int), ("constraints", C.POINTER(C.c_char_p)),
                ("nlookups", C.c_int), ("lookups", C.POINTER(_DomainLookup))]


KINDS = {"full": 0, "row": 1, "col": 2}


class Domain:
    """The reference's (make-domain :name :n :blocks :merge :columns :constraints :lookups), src/domain.lisp:39-53.

    columns: (name, kind, c, shared, data) with kind "full", "row" or "col" and data a vector of base elements;
    constraints: forms as text; lookups: dicts with "tag", "values" (forms) and optionally "num".
    """

    def __init__(self, name, n, blocks=1, merge=False, columns=(), constraints=(), lookups=()):
        self.name, self.n, self.blocks, self.merge = name, n, blocks, merge
        self.columns = [(nm, kind, c, shared, _u32(data)) for nm, kind, c, shared, data in columns]
        self.constraints, self.lookups = list(constraints), list(lookups)
        self._keep = []
        cols = (_DomainColumn * max(len(self.columns), 1))()
        for i, (nm, kind, c, shared, data) in enumerate(self.columns):
            cols[i] = _DomainColumn(nm.encode(), KINDS[kind], c, 1 if shared else 0, _ptr(data))
        cons = _strs(self.constraints)
        looks = (_DomainLookup * max(len(self.lookups), 1))()
        for i, lk in enumerate(self.lookups):
            vals = _strs(list(lk.get("values", [])))
            self._keep.append(vals)
            looks[i] = _DomainLookup(lk["tag"].encode(), len(lk.get("values", [])), vals, lk["num"].encode() if lk.get("num") is not None else None)
        self._keep += [cols, cons, looks]
        self.struct = _Domain(name.encode(), n, blocks, 1 if merge else 0, len(self.columns), cols, len(self.constraints), cons,
                              len(self.lookups), looks)

    def statement(self):
        """(statement text, number of tables, degree, degree of the block phase): DOMAIN-STATEMENT, DOMAIN-TABLES, DOMAIN-DEGREE."""
        buf = C.create_string_buffer(1 << 16)
        nt, deg, bdeg = C.c_int(), C.c_int(), C.c_int()
        _check(library().sc_domain_statement(C.byref(self.struct), buf, C.c_size_t(1 << 16), C.byref(nt), C.byref(deg), C.byref(bdeg)))
        return buf.value.decode(), nt.value, deg.value, bdeg.value


_domain_provers = []


def prove_domain(tr, domain, z, betas, label="dom", provers=None):
    """The reference's (prove-domain tr domain z betas :label label), src/domain.lisp:336-372.

    Returns the column claims, a list of (name, point, value): value is one element when the domain is merged,
    else a list of the blocks' elements (one for a shared column).
    """
    D = tr.degree
    need = max(1, len(domain.lookups))
    if provers is None:
        while len(_domain_provers) < need:
            _domain_provers.append(Prover(0))
        provers = _domain_provers[:need]
    lk = (domain.blocks - 1).bit_length()
    ncol, K, n = len(domain.columns), domain.blocks, domain.n
    za = _u32(z)
    ba = _u32(betas).reshape(-1, D)
    point_len = (C.c_int * ncol)()
    value_rows = (C.c_int * ncol)()
    points = np.zeros((ncol, n + lk, D), dtype=np.uint32)
    values = np.zeros((ncol, K, D), dtype=np.uint32)
    ctxs = (C.c_void_p * len(provers))(*[p._h.value for p in provers])
    rc = library().sc_prove_domain(ctxs, len(provers), C.c_void_p(tr._h), C.byref(domain.struct), _ptr(za), _ptr(ba), len(ba), label.encode(),
                                   point_len, _ptr(points), value_rows, _ptr(values))
    if rc:
        for p in provers:
            if library().sc_last_error(p._h).decode():
                _check(rc, p._h)
        _check(rc)
    out = []
    for i, (name, _, _, shared, _) in enumerate(domain.columns):
        vals = values[i, :value_rows[i]].tolist()
        out.append((name.lower(), points[i, :point_len[i]].tolist(), vals[0] if domain.merge else vals))
    return out
