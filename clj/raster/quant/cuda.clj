(ns raster.quant.cuda
  "CUDA methods of the quantized-matmul operators: the SAME generic functions as
  raster.quant.op / raster.quant.train / raster.quant.kernels-k / raster.quant.core, extended with
  methods that run on librstq (B200).  `deftm` is multiple dispatch (src/raster/core.clj:597-638):
  a second method on other argument types from another namespace extends the existing function, so
  callers keep calling `qlinear-i8` and the placement policy decides where it runs.

  Two routes, as the boundary asks:
   * JVM arrays in, JVM arrays out (the literal drop-in): the weight is uploaded and re-tiled the
     first time its arrays are seen and stays resident; only x and y cross PCIe;
   * device-resident `QWeight` + buffer records (the resident-program path): nothing but the launch."
  (:require [raster.core :refer [deftm]]
            [raster.compiler.core.op-descriptor :as descriptor]
            [raster.gpu.cuda-runtime :as rt])
  (:import [java.lang.foreign Arena MemorySegment ValueLayout]))

(defn- seg ^MemorySegment [arr] (MemorySegment/ofArray arr))
(defn- ctx [] (:ctx (rt/init!)))

;; ---------------------------------------------------------------------------
;; Operator API: same arities as src/raster/quant/op.clj:43-99
;; ---------------------------------------------------------------------------

(deftm ^:no-inline raster.quant.op/qlinear-i8!
  "qlinear-i8! on :cuda:N -- W4A8: x quantized to int8 blocks on the device, integer block dots,
  per-block scale fold; y fully overwritten."
  [x :- (Array float), wqi :- (Array byte), wsi :- (Array float),
   y :- (Array float), in :- Long, out :- Long] :- (Array float)
  (rt/rstq! "rstq_qlinear_i8"
            (.invokeWithArguments @#'rt/qlinear-i8* (object-array [(ctx) (seg x) (seg wqi) (seg wsi) (seg y) (long in) (long out)])))
  y)

(deftm raster.quant.op/qlinear-i8
  [x :- (Array float), wqi :- (Array byte), wsi :- (Array float), in :- Long, out :- Long] :- (Array float)
  (let [y (float-array out)]
    (raster.quant.op/qlinear-i8! x wqi wsi y in out)
    y))

(deftm ^:no-inline raster.quant.op/qlinear-i8-q8!
  [x :- (Array float), wqi :- (Array byte), wsi :- (Array float),
   y :- (Array float), in :- Long, out :- Long] :- (Array float)
  (rt/rstq! "rstq_qlinear_i8_q8"
            (.invokeWithArguments @#'rt/qlinear-i8-q8* (object-array [(ctx) (seg x) (seg wqi) (seg wsi) (seg y) (long in) (long out)])))
  y)

(deftm raster.quant.op/qlinear-i8-q8
  [x :- (Array float), wqi :- (Array byte), wsi :- (Array float), in :- Long, out :- Long] :- (Array float)
  (let [y (float-array out)]
    (raster.quant.op/qlinear-i8-q8! x wqi wsi y in out)
    y))

;; src/raster/quant/train.clj:77-108 -- W8A32 with an M dimension
(deftm ^:no-inline raster.quant.train/qlinear-q8
  [x :- (Array float), codes :- (Array byte), scales :- (Array float),
   m :- Long, in :- Long, out :- Long] :- (Array float)
  (let [y (float-array (* m out))]
    (rt/rstq! "rstq_qlinear_q8"
              (.invokeWithArguments @#'rt/qlinear-q8* (object-array [(ctx) (seg x) (seg codes) (seg scales) (seg y) (long m) (long in) (long out)])))
    y))

;; src/raster/quant/train.clj:110-137
(deftm ^:no-inline raster.quant.train/qlinear-q8-dx
  [dy :- (Array float), codes :- (Array byte), scales :- (Array float),
   m :- Long, in :- Long, out :- Long] :- (Array float)
  (let [dx (float-array (* m in))]
    (rt/rstq! "rstq_qlinear_q8_dx"
              (.invokeWithArguments @#'rt/qlinear-q8-dx* (object-array [(ctx) (seg dy) (seg codes) (seg scales) (seg dx) (long m) (long in) (long out)])))
    dx))

;; src/raster/quant/kernels_k.clj:344-370 -- prefill W8A8, acts already quantized per (row, block)
(deftm ^:no-inline raster.quant.kernels-k/qmatmul-i8-gemm!
  [xp :- (Array int), xs :- (Array float), wp :- (Array int), ws :- (Array float),
   y :- (Array float), in :- Long, out :- Long, nrows :- Long] :- (Array float)
  (rt/rstq! "rstq_qmatmul_i8_gemm"
            (.invokeWithArguments @#'rt/qmatmul-i8-gemm* (object-array [(ctx) (seg xp) (seg xs) (seg wp) (seg ws) (seg y) (long in) (long out) (long nrows)])))
  y)

;; ---------------------------------------------------------------------------
;; Resident path: a bound weight and buffer records (rt/make-buffer)
;; ---------------------------------------------------------------------------

(defrecord QWeight [handle rows cols format device])

(def formats {:q4-0 0 :q8-0 1 :q8-signed 2})
(def layouts {:row-major 0 :stream8 1})

(defn bind-weight
  "Uploads and re-tiles a weight in one of the reference's host layouts (load time, replaces
  repack-stream as the load-time transform).  `shard` = nil or {:split :column|:row :rank r :ranks P}."
  [codes scales rows cols fmt layout dev shard]
  (with-open [a (Arena/ofConfined)]
    (let [out (.allocate a ValueLayout/ADDRESS)]
      (if shard
        (rt/rstq! "rstq_weight_bind_shard"
                  (.invokeWithArguments @#'rt/weight-bind-shard*
                                        (object-array [(ctx) out (seg codes) (seg scales) (int dev) (long rows) (long cols)
                                                       (int (formats fmt)) (int (layouts layout))
                                                       (int ({:column 1 :row 2} (:split shard))) (int (:rank shard)) (int (:ranks shard))])))
        (rt/rstq! "rstq_weight_bind"
                  (.invokeWithArguments @#'rt/weight-bind*
                                        (object-array [(ctx) out (seg codes) (seg scales) (int dev) (long rows) (long cols)
                                                       (int (formats fmt)) (int (layouts layout))]))))
      (->QWeight (.get out ValueLayout/ADDRESS 0) rows cols fmt dev))))

(defn qmatmul!
  "One kernel step of a resident program: y[M, rows] = W . x[M, cols] on device buffers.
  `mode` :a8 = qlinear-i8 arithmetic, :f = float activations times dequantized weights."
  [^QWeight w x y m mode]
  (rt/rstq! "rstq_qmatmul"
            (.invokeWithArguments @#'rt/qmatmul*
                                  (object-array [(ctx) (:handle w) (:segment x) (:segment y) (long m)
                                                 (int (if (= :bf16 (:dtype x)) rt/RSTQ_BF16 rt/RSTQ_F32))
                                                 (int (if (= :bf16 (:dtype y)) rt/RSTQ_BF16 rt/RSTQ_F32))
                                                 (int (if (= mode :a8) rt/RSTQ_MODE_A8 rt/RSTQ_MODE_F))])))
  y)

;; the operator names a chain program refers to (gpu/core.clj chain-program!, :711-767)
(rt/register-kernel! "qmatmul-q4-x8!" (fn [w xq xs xsum y m]
                                        (rt/rstq! "rstq_qmatmul_prequant"
                                                  (.invokeWithArguments @#'rt/qmatmul-prequant*
                                                                        (object-array [(ctx) (:handle w) (:segment xq) (:segment xs)
                                                                                       (:segment xsum) (:segment y) (long m)])))))

;; ---------------------------------------------------------------------------
;; Op-descriptor facets for the CUDA methods (the CPU ones: src/raster/quant/op.clj:68-79, 101-119)
;; ---------------------------------------------------------------------------

;; buffer semantics are a property of the generic function and stay as registered by raster.quant.op:
;; qlinear-i8 allocates float-array[out] and is rewritten to the ! form, which fully overwrites
;; argument 3.  The CUDA kernels store every y exactly once and never read it: the same contract.
(descriptor/register-buffer-write! 'raster.quant.op/qlinear-i8!    :overwrite 3)
(descriptor/register-buffer-write! 'raster.quant.op/qlinear-i8-q8! :overwrite 3)
(descriptor/register-op-descriptor! 'raster.quant.op/qlinear-i8!    {:effects {:pure? false :mutating? true}})
(descriptor/register-op-descriptor! 'raster.quant.op/qlinear-i8-q8! {:effects {:pure? false :mutating? true}})

;; placement: a second profile beside :cpu-quant; a policy {:gpu-quant :cuda:0} sends the ops here
;; (src/raster/compiler/passes/placement.clj:21-25; tests override the policy the same way,
;; test/raster/compiler/passes/placement_test.clj:12)
(doseq [op '[raster.quant.op/qlinear-i8 raster.quant.op/qlinear-i8! raster.quant.op/qlinear-i8-q8
             raster.quant.op/qlinear-i8-q8! raster.quant.train/qlinear-q8 raster.quant.train/qlinear-q8-dx
             raster.quant.kernels-k/qmatmul-i8-gemm!]]
  (descriptor/register-placement! op :gpu-quant))

(def default-policy-entry
  "Merge into placement/default-policy to run the quant ops on the first B200."
  {:gpu-quant :cuda:0})
