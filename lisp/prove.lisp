;;;; prove.lisp -- EXACTA.SUMCHECK:PROVE (src/sumcheck.lisp:512-571) with its rounds on the device.
;;;;
;;;; What stays in Lisp: the statement (EXPAND gives the term table), the transcript (header, SEND,
;;;; CHALLENGE) and the shape of the results.  What moves: tables, weights, round sums and folds.

(in-package #:exacta.b200)

(defun u32-vector (n) (make-array n :element-type '(unsigned-byte 32) :initial-element 0))
(defun s32-vector (n) (make-array n :element-type '(signed-byte 32) :initial-element 0))

;;; ------------------------------------------------------------------ tables

(defstruct (flat-table (:constructor make-flat-table (words stride)))
  "A table that is flat already: WORDS is a (simple-array (unsigned-byte 32) (*)) of entries of STRIDE words
(1: base field, else the extension degree).  Passing one in the TABLES alist avoids boxing 2^26 and more entries."
  (words nil :type (simple-array (unsigned-byte 32) (*)))
  (stride 1 :type (integer 1 8)))

(defun flatten-table (values d)
  "VALUES as a flat vector and its stride, as MAKE-TABLE lays it out (src/sumcheck.lisp:61-70)."
  (if (flat-table-p values)
      (values (flat-table-words values) (flat-table-stride values))
      (let ((values (coerce values 'vector)))
        (if (every #'integerp values)
            (values (coerce-ext values) 1)
            (let ((words (u32-vector (* d (length values)))))
              (loop for v across values
                    for x from 0
                    do (replace words (if (integerp v) (base->ext v d) v) :start1 (* d x)))
              (values words d))))))

;;; ------------------------------------------------------------------ the statement as a term table

(defun term-table (statement names constants d)
  "EXPAND's monomials with the constants' values multiplied in and equal table lists merged: a list of
(sorted-table-indices . coefficient EXT), zero terms dropped (what sc_set_statement takes)."
  (let ((terms (make-hash-table :test 'equal)))
    (loop for (monomial . c) in (expand statement)
          do (let ((coefficient (base->ext c d))
                   (indices '()))
               (dolist (variable monomial)
                 (let ((constant (assoc variable constants)))
                   (cond (constant (setf coefficient (ext* coefficient (cdr constant))))
                         ((position variable names) (push (position variable names) indices))
                         (t (error 'invalid-parameter :name 'variable :value variable
                                                      :expected "a table or a constant")))))
               (let ((key (sort indices #'<)))
                 (setf (gethash key terms) (ext+ (gethash key terms (make-ext d)) coefficient)))))
    (loop for key being the hash-keys of terms using (hash-value c)
          unless (every #'zerop c) collect (cons key c))))

(defun set-statement (ctx statement names constants d points)
  (let* ((terms (term-table statement names constants d))
         (coeffs (u32-vector (* d (max 1 (length terms)))))
         (ptr (s32-vector (1+ (length terms))))
         (idx (s32-vector (max 1 (reduce #'+ terms :key (lambda (term) (length (car term))))))))
    (loop with at = 0
          for (indices . c) in terms
          for i from 0
          do (replace coeffs c :start1 (* d i))
             (setf (aref ptr i) at)
             (dolist (index indices) (setf (aref idx at) index) (incf at))
          finally (setf (aref ptr (length terms)) at))
    (with-saps ((c coeffs) (p ptr) (x idx))
      (check (%set-statement ctx d points (length names) (length terms) c p x) ctx))))

;;; ------------------------------------------------------------------ the transcript's hash state, for the device

(defun attach-transcript-state (ctx tr)
  "Hand the B3S state of TR (src/blake3.lisp:125-131) to the library, for a chain of rounds that starts now."
  (let* ((state (transcript-state tr))
         (cv (coerce (exacta.blake3::b3s-cv state) '(simple-array (unsigned-byte 32) (*))))
         (block (exacta.blake3::b3s-block state))
         (pending (u32-vector 16)))
    (dotimes (i 16) (setf (aref pending i) (le-integer block (* 4 i) 4)))
    (with-saps ((c cv) (p pending))
      (check (%attach-transcript-state ctx c p (exacta.blake3::b3s-used state) (exacta.blake3::b3s-counter state)) ctx))))

;;; ------------------------------------------------------------------ PROVE

(defun concatenate-exts (exts count)
  (let ((exts (coerce exts 'vector)))
    (when (plusp count)
      (let* ((d (length (aref exts 0)))
             (out (u32-vector (* d count))))
        (dotimes (i count out) (replace out (aref exts i) :start1 (* d i)))))))

(defun prove (tr n statement tables &key eq constants (label "sc") block-weights
                                      (degree (exacta.sumcheck:statement-degree statement constants)))
  "EXACTA.SUMCHECK:PROVE with the same arguments and the same three values -- the round challenges, the finals
and the folded tables -- and TR left with the same messages and state.  A table may also be a FLAT-TABLE."
  (let* ((d (transcript-degree tr))
         (points (max degree 1))
         (names (mapcar #'car tables))
         (k (if block-weights (length block-weights) 1))
         (ctx (context)))
    (set-statement ctx statement names constants d points)
    (loop for (nil . values) in tables
          for slot from 0
          do (multiple-value-bind (words stride) (flatten-table values d)
               (with-saps ((h words))
                 (check (%upload-table ctx slot h (floor (length words) stride) stride) ctx))))
    (with-saps ((e (and eq (concatenate-exts eq n)))
                (b (and block-weights (concatenate-exts block-weights k))))
      (check (%begin ctx n e k b) ctx))
    (absorb tr (exacta.sumcheck:header label n degree k))
    (let ((sums (u32-vector (* points d)))
          (rhos '()))
      (dotimes (j n)
        (when *device-transcript* (attach-transcript-state ctx tr))
        (with-saps ((s sums)) (check (%round ctx s) ctx))
        (let ((message (make-array (list points d) :element-type '(unsigned-byte 32))))
          (dotimes (i (* points d)) (setf (row-major-aref message i) (aref sums i)))
          (send tr message))
        (let ((r (challenge tr)))
          (push r rhos)
          (with-saps ((rs r)) (check (%challenge ctx rs) ctx))))
      (let ((folded (u32-vector (* (length names) k d))))
        (with-saps ((f folded)) (check (%finish ctx f) ctx))
        (flet ((entry (table block)
                 (let ((out (make-ext d)))
                   (replace out folded :start2 (* d (+ (* table k) block)))
                   out)))
          (values (nreverse rhos)
                  (loop for name in names
                        for i from 0
                        collect (cons name (entry i 0)))
                  (loop for name in names
                        for i from 0
                        collect (cons name (coerce (loop for b below k collect (entry i b)) 'vector)))))))))

;;; ------------------------------------------------------------------ putting it under the reference's callers

(defvar *reference-prove* nil "EXACTA.SUMCHECK:PROVE as it was before INSTALL.")

(defun install ()
  "Make EXACTA.SUMCHECK:PROVE run on the device."
  (unless *reference-prove*
    (setf *reference-prove* (fdefinition 'exacta.sumcheck:prove)))
  (setf (fdefinition 'exacta.sumcheck:prove) #'prove)
  t)

(defun uninstall ()
  "Put the Lisp prover back."
  (when *reference-prove*
    (setf (fdefinition 'exacta.sumcheck:prove) *reference-prove*
          *reference-prove* nil))
  t)
