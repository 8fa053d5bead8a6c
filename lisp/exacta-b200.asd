;;;; exacta-b200.asd -- Exacta's sumcheck prover with its rounds on a B200 (libsumcheck_b200.so).
;;;;
;;;; Load after "exacta".  (exacta.b200:install) makes EXACTA.SUMCHECK:PROVE run on the device, so the
;;;; callers (PROVE-UPPER, PROVE-DOMAIN, REDUCE-POINTS) and the reference's own tests go through it
;;;; unchanged; (exacta.b200:uninstall) puts the Lisp prover back.
;;;;
;;;; Untested: no Common Lisp was available where this was written.  The C functions it binds are
;;;; tested through the same ABI from Python.

(defsystem "exacta-b200"
  :description "EXACTA.SUMCHECK:PROVE on a B200: the prover rounds as CUDA kernels behind a C ABI."
  :version "0.2.0"
  :license "MIT"
  :depends-on ("exacta")
  :serial t
  :components ((:file "package")
               (:file "ffi")
               (:file "prove")))
