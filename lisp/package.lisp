;;;; package.lisp -- the package of the B200 prover.

(defpackage #:exacta.b200
  (:use #:cl #:exacta.util #:exacta.conditions #:exacta.field #:exacta.forms #:exacta.transcript)
  (:export #:prove #:install #:uninstall
           #:*library* #:*device* #:*context* #:*device-transcript*
           #:make-context #:destroy-context #:flat-table #:make-flat-table #:device-error))

(in-package #:exacta.b200)

(defvar *library* "libsumcheck_b200.so"
  "The shared library, as LOAD-SHARED-OBJECT finds it (a full path, or a name on the loader's path).")
(defvar *device* 0 "The CUDA device ordinal of the context made on first use.")
(defvar *context* nil "The device context (a system area pointer), made on first use.")
(defvar *device-transcript* nil
  "True: the round kernels carry the transcript on themselves (all rounds enqueued at once); PROVE replays
SEND and CHALLENGE on the Lisp transcript and the library checks that they agree.")
