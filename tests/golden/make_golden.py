#!/usr/bin/env python3
"""Regenerate tests/golden/vectors.json from the reference's known-answer vectors.

The reference keeps its known-answer tests in one s-expression file, tests/vectors.sexp
(written by the original Python implementation).  The kinds that pin the sumcheck prover path are
copied here, as data, into JSON so that the tests run where the reference tree is not mounted:

  :ext :lagrange :eq :mle :pow   field and tower arithmetic      (vectors.sexp:4-52)
  :b3s                           sequential BLAKE3               (vectors.sexp:72-77)
  :transcript                    Fiat-Shamir transcript          (vectors.sexp:78)
  :proofio                       proof bytes                     (vectors.sexp:89)
  :poly                          expansion of a form             (vectors.sexp:97)
  :sumcheck                      whole proofs                    (vectors.sexp:103-106)

Usage:  python tests/golden/make_golden.py [path/to/vectors.sexp]
"""
import json
import os
import re
import sys

KEEP = (":ext", ":lagrange", ":eq", ":mle", ":pow", ":b3s", ":transcript", ":proofio", ":poly",
        ":sumcheck")


def parse(text):
    tokens = re.findall(r'\(|\)|"[^"]*"|[^\s()]+', text)
    pos = 0

    def read():
        nonlocal pos
        tok = tokens[pos]
        pos += 1
        if tok == "(":
            out = []
            while tokens[pos] != ")":
                out.append(read())
            pos += 1
            return out
        if tok.startswith('"'):
            return {"str": tok[1:-1]}
        if tok.lower() == "nil":
            return None
        if tok.lower() == "t":
            return True
        try:
            return int(tok)
        except ValueError:
            return tok

    return read()


def unstring(x):
    if isinstance(x, dict):
        return x["str"]
    if isinstance(x, list):
        return [unstring(y) for y in x]
    return x


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <reference tree>/tests/vectors.sexp")
    src = sys.argv[1]
    text = "\n".join(line for line in open(src).read().split("\n") if not line.startswith(";"))
    out = {}
    for vector in parse(text):
        kind = vector[0]
        if kind not in KEEP:
            continue
        fields = {}
        for i in range(1, len(vector), 2):
            fields[vector[i].lstrip(":")] = unstring(vector[i + 1])
        out.setdefault(kind.lstrip(":"), []).append(fields)
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "vectors.json"), "w") as f:
        json.dump(out, f, separators=(",", ":"))
        f.write("\n")
    print({k: len(v) for k, v in out.items()})


if __name__ == "__main__":
    main()
