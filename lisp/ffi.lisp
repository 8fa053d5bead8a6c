;;;; ffi.lisp -- the C ABI of include/sumcheck_b200.h, part 1 (the device layer), through sb-alien.
;;;;
;;;; Every routine returns 0 or a negative SC_E* code.  Vectors are passed as system area pointers of
;;;; pinned (unsigned-byte 32) or (signed-byte 32) vectors (WITH-SAPS); a NIL vector becomes a null pointer.

(in-package #:exacta.b200)

(defvar *loaded* nil)
(defun ensure-library ()
  (unless *loaded*
    (sb-alien:load-shared-object *library*)
    (setf *loaded* t)))

(defmacro define-sc (c-name lisp-name &rest arguments)
  "An alien routine returning int."
  `(sb-alien:define-alien-routine (,c-name ,lisp-name) sb-alien:int ,@arguments))

(define-sc "sc_create" %create (device sb-alien:int) (ctx (* sb-alien:system-area-pointer)))
(define-sc "sc_destroy" %destroy (ctx sb-alien:system-area-pointer))
(define-sc "sc_set_memory_budget" %set-memory-budget (ctx sb-alien:system-area-pointer) (bytes (sb-alien:unsigned 64)))
(define-sc "sc_set_statement" %set-statement
  (ctx sb-alien:system-area-pointer) (d sb-alien:int) (points sb-alien:int) (ntables sb-alien:int) (nterms sb-alien:int)
  (coeffs sb-alien:system-area-pointer) (term-ptr sb-alien:system-area-pointer) (term-tables sb-alien:system-area-pointer))
(define-sc "sc_upload_table" %upload-table
  (ctx sb-alien:system-area-pointer) (slot sb-alien:int) (host sb-alien:system-area-pointer)
  (entries (sb-alien:unsigned 64)) (stride sb-alien:int))
(define-sc "sc_begin" %begin
  (ctx sb-alien:system-area-pointer) (n sb-alien:int) (eq sb-alien:system-area-pointer) (k sb-alien:int)
  (block-weights sb-alien:system-area-pointer))
(define-sc "sc_round" %round (ctx sb-alien:system-area-pointer) (sums sb-alien:system-area-pointer))
(define-sc "sc_challenge" %challenge (ctx sb-alien:system-area-pointer) (r sb-alien:system-area-pointer))
(define-sc "sc_finish" %finish (ctx sb-alien:system-area-pointer) (folded sb-alien:system-area-pointer))
(define-sc "sc_set_device_transcript" %set-device-transcript (ctx sb-alien:system-area-pointer) (on sb-alien:int))
(define-sc "sc_attach_transcript_state" %attach-transcript-state
  (ctx sb-alien:system-area-pointer) (cv sb-alien:system-area-pointer) (pending sb-alien:system-area-pointer)
  (fill sb-alien:int) (blocks (sb-alien:unsigned 64)))
(sb-alien:define-alien-routine ("sc_last_error" %last-error) sb-alien:c-string (ctx sb-alien:system-area-pointer))
(sb-alien:define-alien-routine ("sc_strerror" %strerror) sb-alien:c-string (code sb-alien:int))

(define-condition device-error (exacta-error)
  ((code :initarg :code :reader device-error-code)
   (text :initarg :text :reader device-error-text))
  (:report (lambda (c stream)
             (format stream "libsumcheck_b200: ~A (code ~D)" (device-error-text c) (device-error-code c))))
  (:documentation "A failure inside the library that is not the caller's argument: CUDA, memory, the collective layer."))

(defun check (code ctx)
  "0, or the reference's conditions: INVALID-PARAMETER for bad arguments (SC_EINVAL, SC_ESTATEMENT), else DEVICE-ERROR."
  (unless (zerop code)
    (let ((text (if ctx (%last-error ctx) (%strerror code))))
      (if (member code '(-1 -7))
          (error 'invalid-parameter :name 'sumcheck :value code :expected text)
          (error 'device-error :code code :text text)))))

(defun null-sap () (sb-sys:int-sap 0))

(defmacro with-saps ((&rest bindings) &body body)
  "BINDINGS: (sap vector-form).  Pin the vectors (never WITHOUT-GCING) and bind their system area pointers; a
vector-form that gives NIL binds a null pointer."
  (let ((vectors (loop for nil in bindings collect (gensym "VECTOR"))))
    `(let ,(loop for (nil form) in bindings for v in vectors collect `(,v ,form))
       (sb-sys:with-pinned-objects ,vectors
         (let ,(loop for (sap nil) in bindings for v in vectors
                     collect `(,sap (if ,v (sb-sys:vector-sap ,v) (null-sap))))
           ,@body)))))

(defun make-context (&optional (device *device*))
  "A device context on CUDA device DEVICE; DESTROY-CONTEXT (or the finalizer) gives its memory back."
  (ensure-library)
  (let ((ctx (sb-alien:with-alien ((out sb-alien:system-area-pointer))
               (check (%create device (sb-alien:addr out)) nil)
               out)))
    (when *device-transcript* (check (%set-device-transcript ctx 1) ctx))
    ctx))

(defun destroy-context (&optional (ctx *context*))
  (when ctx
    (%destroy ctx)
    (when (eq ctx *context*) (setf *context* nil))))

(defun context ()
  (or *context* (setf *context* (make-context))))
