"""The Lisp side of the boundary (lisp/*.lisp, lisp/exacta-b200.asd), checked without a Lisp.

No Common Lisp is installed where the tests run, so the files cannot be loaded.  What can be checked by
reading them: every form is balanced and readable, every C function they bind is declared in
include/sumcheck_b200.h with the same number of arguments, the files the system names exist, and PROVE
has the reference's lambda list (src/sumcheck.lisp:512-513)."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LISP = os.path.join(ROOT, "lisp")


def read_forms(text):
    """A small s-expression reader: lists, strings, symbols, numbers, quote-like prefixes, ; and #| |# comments."""
    pos, n = 0, len(text)

    def skip():
        nonlocal pos
        while pos < n:
            c = text[pos]
            if c.isspace():
                pos += 1
            elif c == ";":
                while pos < n and text[pos] != "\n":
                    pos += 1
            elif text.startswith("#|", pos):
                end = text.index("|#", pos)
                pos = end + 2
            else:
                break

    def read():
        nonlocal pos
        skip()
        if pos >= n:
            raise EOFError
        c = text[pos]
        if c == "(":
            pos += 1
            out = []
            while True:
                skip()
                if pos >= n:
                    raise SyntaxError("unbalanced: a list is never closed")
                if text[pos] == ")":
                    pos += 1
                    return out
                out.append(read())
        if c == ")":
            raise SyntaxError("unbalanced: ) at offset %d" % pos)
        if c == '"':
            end = pos + 1
            while text[end] != '"':
                end += 2 if text[end] == "\\" else 1
            s = text[pos + 1:end]
            pos = end + 1
            return ("string", s)
        for prefix in ("#'", "#:", ",@", "'", "`", ",", "#."):
            if text.startswith(prefix, pos):
                pos += len(prefix)
                return [("prefix", prefix), read()] if prefix != "#:" else read()
        if text.startswith("#\\", pos):
            pos += 3
            while pos < n and (text[pos].isalnum() or text[pos] == "-"):
                pos += 1
            return ("char",)
        end = pos
        while end < n and not text[end].isspace() and text[end] not in "()\"":
            end += 1
        token = text[pos:end]
        pos = end
        return token.lower()

    forms = []
    while True:
        try:
            forms.append(read())
        except EOFError:
            return forms


def header_functions():
    text = open(os.path.join(ROOT, "include", "sumcheck_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = {}
    for m in re.finditer(r"\b(sc_[a-z0-9_]+)\s*\(([^;{}]*?)\)\s*;", text):
        params = m.group(2).strip()
        out[m.group(1)] = 0 if params in ("", "void") else len(params.split(","))
    return out


def walk(form):
    yield form
    if isinstance(form, list):
        for f in form:
            yield from walk(f)


def lisp_files():
    return sorted(f for f in os.listdir(LISP) if f.endswith((".lisp", ".asd")))


def test_every_form_reads_and_is_balanced():
    assert "exacta-b200.asd" in lisp_files() and "prove.lisp" in lisp_files()
    for name in lisp_files():
        forms = read_forms(open(os.path.join(LISP, name)).read())
        assert forms, name
        assert all(isinstance(f, list) for f in forms), "%s: a stray atom at top level" % name


def test_the_system_names_files_that_exist():
    (system,) = [f for f in read_forms(open(os.path.join(LISP, "exacta-b200.asd")).read()) if f[0] == "defsystem"]
    assert ("string", "exacta") in system[system.index(":depends-on") + 1]
    components = system[system.index(":components") + 1]
    for kind, (_, name) in components:
        assert kind == ":file" and os.path.exists(os.path.join(LISP, name + ".lisp")), name


def test_bound_c_functions_match_the_header():
    declared = header_functions()
    bound = {}
    for name in lisp_files():
        for form in walk(read_forms(open(os.path.join(LISP, name)).read())):
            if isinstance(form, list) and form and form[0] == "define-sc" and len(form) > 2 and isinstance(form[1], tuple):
                bound[form[1][1]] = len(form) - 3                  # (define-sc "c_name" lisp-name (arg type)...)
            if isinstance(form, list) and form and form[0] == "sb-alien:define-alien-routine" and isinstance(form[1], list) \
                    and form[1] and isinstance(form[1][0], tuple):
                bound[form[1][0][1]] = len(form) - 3               # (define-alien-routine ("c_name" lisp-name) result (arg type)...)
    assert {"sc_create", "sc_destroy", "sc_set_statement", "sc_upload_table", "sc_begin", "sc_round", "sc_challenge", "sc_finish",
            "sc_last_error"} <= set(bound)
    for c_name, nargs in bound.items():
        assert c_name in declared, "%s is bound but not declared in the header" % c_name
        assert declared[c_name] == nargs, "%s: the header has %d arguments, the binding %d" % (c_name, declared[c_name], nargs)


def test_prove_has_the_reference_lambda_list():
    forms = read_forms(open(os.path.join(LISP, "prove.lisp")).read())
    (prove,) = [f for f in forms if f[:2] == ["defun", "prove"]]
    names = [p if isinstance(p, str) else p[0] for p in prove[2]]
    assert names == ["tr", "n", "statement", "tables", "&key", "eq", "constants", "label", "block-weights", "degree"]
    label = [p for p in prove[2] if isinstance(p, list) and p[0] == "label"][0]
    assert label[1] == ("string", "sc")
    defined = {f[1] for f in forms if isinstance(f, list) and f[0] == "defun"}
    assert {"install", "uninstall", "prove"} <= defined
    # every helper PROVE calls from this package is defined in one of the files
    everything = set()
    for name in lisp_files():
        for f in read_forms(open(os.path.join(LISP, name)).read()):
            if isinstance(f, list) and f and f[0] in ("defun", "defmacro", "defstruct", "define-sc"):
                target = f[2] if f[0] == "define-sc" else f[1]
                everything.add(target[0] if isinstance(target, list) else target)
    for helper in ("context", "set-statement", "flatten-table", "concatenate-exts", "attach-transcript-state", "check", "with-saps",
                   "%upload-table", "%begin", "%round", "%challenge", "%finish", "u32-vector", "make-context", "null-sap"):
        assert helper in everything, helper
