(ns raster.gpu.cuda-runtime
  "The CUDA runtime namespace the session layer resolves by name
  (src/raster/gpu/core.clj:39-84 looks the functions below up in the namespace `backend-ns`
  returns): buffers, bound launches, graphs, events -- all through librstq's C ABI
  (include/rstq.h), bound with Panama FFM exactly as the OpenCL runtime binds its driver
  (src/raster/gpu/ocl_runtime.clj:59-76, 192-199).

  Every native function is declared ONCE, with `defrstq`:

      (defrstq handle-var \"c_symbol\" RET [ARG ...])

  RET / ARG are the one-letter layouts below.  tests/test_clj_binding.py parses these forms and
  checks each against the prototype in include/rstq.h (arity, pointer / scalar kind and order),
  so the table cannot drift from the header.  No JVM exists where this repository is built and
  tested: the file is the binding a Raster maintainer adds, kept honest by that check and by the
  ctypes twin (raster_b200/_lib.py) that drives the same entry points in the same argument order."
  (:import [java.lang.foreign Arena FunctionDescriptor Linker Linker$Option MemoryLayout
            MemorySegment SymbolLookup ValueLayout]))

;; ---------------------------------------------------------------------------
;; Loading, layouts, the status wrapper
;; ---------------------------------------------------------------------------

(def ^:private I ValueLayout/JAVA_INT)      ; int32_t
(def ^:private L ValueLayout/JAVA_LONG)     ; int64_t
(def ^:private F ValueLayout/JAVA_FLOAT)    ; float
(def ^:private D ValueLayout/JAVA_DOUBLE)   ; double
(def ^:private P ValueLayout/ADDRESS)       ; any pointer / opaque handle

(defonce ^:private lib
  (delay (SymbolLookup/libraryLookup (or (System/getenv "RASTER_RSTQ_LIB") "librstq.so") (Arena/global))))
(def ^:private lnk (Linker/nativeLinker))

(defn- downcall [sym ret args]
  (.downcallHandle lnk (.orElseThrow (.find ^SymbolLookup @lib sym))
                   (FunctionDescriptor/of ret (into-array MemoryLayout args))
                   (into-array Linker$Option [])))

(defmacro defrstq
  "Declares `nm` as the (delayed) downcall handle of C function `sym`."
  [nm sym ret args]
  `(def ~(with-meta nm {:private true}) (delay (downcall ~sym ~ret ~args))))

;; ---- library / errors
(defrstq version*            "rstq_version"        I [])
(defrstq last-error*         "rstq_last_error"     P [])
(defrstq device-count*       "rstq_device_count"   I [P])
;; ---- context
(defrstq init*               "rstq_init"           I [P P I])        ; devices ctx** ndev
(defrstq shutdown*           "rstq_shutdown"       I [P])
(defrstq sync*               "rstq_sync"           I [P I])          ; ctx dev
(defrstq gemm-plan*          "rstq_gemm_plan"      I [P L L L I])    ; plan2 out in m sm-count
(defrstq decode-plan*        "rstq_decode_plan"    I [P I I L L L I I])  ; plan6 mode bits out in m act-dtype sm-count
(defrstq tune*               "rstq_tune"           I [P I L])        ; ctx key value
(defrstq device-info*        "rstq_device_info"    I [P P I])        ; ctx out4 dev
(defrstq timeline-read*      "rstq_timeline_read"  I [P P I L])      ; ctx out dev n
;; ---- device buffers
(defrstq alloc*              "rstq_alloc"          I [P P I L])      ; ctx buf** dev bytes
(defrstq free*               "rstq_free"           I [P])
(defrstq upload*             "rstq_upload"         I [P P L L])      ; buf host offset bytes
(defrstq download*           "rstq_download"       I [P P L L])
(defrstq memset*             "rstq_memset"         I [P I L L])      ; buf byte offset bytes
(defrstq buf-ptr*            "rstq_buf_ptr"        I [P P P])
(defrstq buf-wrap*           "rstq_buf_wrap"       I [P P P I L])    ; ctx buf** device-ptr dev bytes
(defrstq stream-set*         "rstq_stream_set"     I [P P I])        ; ctx stream dev
;; ---- weights
(defrstq weight-bind*        "rstq_weight_bind"       I [P P P P I L L I I])       ; ctx w** codes scales dev out in fmt layout
(defrstq weight-bind-shard*  "rstq_weight_bind_shard" I [P P P P I L L I I I I I]) ; ... split rank nranks
(defrstq weight-bind-q4k*    "rstq_weight_bind_q4k"   I [P P P P P P P I L L])     ; ctx w** wq da db aq bq dev out in
(defrstq weight-bind-q6k*    "rstq_weight_bind_q6k"   I [P P P P P I L L])         ; ctx w** wq sc ds dev out in
(defrstq weight-clone*       "rstq_weight_clone"      I [P P])
(defrstq weight-free*        "rstq_weight_free"       I [P])
(defrstq weight-info*        "rstq_weight_info"       I [P P])
(defrstq weight-cache-clear* "rstq_weight_cache_clear" I [P])
;; ---- device-resident operators (the kernel steps of a resident program)
(defrstq quant-act-i8*       "rstq_quant_act_i8"      I [P P P P P L L])           ; ctx x xq xs xsum M in
(defrstq quant-act-q8k*      "rstq_quant_act_q8k"     I [P P P P P L L I])         ; ctx x xq xs bsums rows in sub
(defrstq qmatmul*            "rstq_qmatmul"           I [P P P P L I I I])         ; ctx w x y M act out mode
(defrstq qmatmul-prequant*   "rstq_qmatmul_prequant"  I [P P P P P P L])           ; ctx w xq xs xsum y M
(defrstq qmatmul-prequant-noalloc* "rstq_qmatmul_prequant_noalloc" I [P P P P P P L]) ; w xq xs xsum y stream M
(defrstq qlinear-q8-dx-device* "rstq_qlinear_q8_dx_device" I [P P P P P L L L])    ; ctx dy codes scales dx m in out
;; ---- host-array operators (JVM arrays in, JVM arrays out)
(defrstq qlinear-i8*         "rstq_qlinear_i8"        I [P P P P P L L])           ; ctx x wqi wsi y in out
(defrstq qlinear-i8-q8*      "rstq_qlinear_i8_q8"     I [P P P P P L L])
(defrstq qlinear-q8*         "rstq_qlinear_q8"        I [P P P P P L L L])         ; ctx x codes scales y m in out
(defrstq qlinear-q8-dx*      "rstq_qlinear_q8_dx"     I [P P P P P L L L])         ; ctx dy codes scales dx m in out
(defrstq qmatmul-i8-gemm*    "rstq_qmatmul_i8_gemm"   I [P P P P P P L L L])       ; ctx xp xs wp ws y in out nrows
(defrstq i8gemv-dp4a*        "rstq_i8gemv_dp4a"       I [P P P P L L])             ; ctx wp xp y kw out
(defrstq qmatmul-host*       "rstq_qmatmul_host"      I [P P P P L I I])           ; ctx w x y M act mode
;; ---- graphs / events
(defrstq graph-begin*        "rstq_graph_begin"       I [P I])
(defrstq graph-end*          "rstq_graph_end"         I [P P I])                   ; ctx graph** dev
(defrstq graph-replay*       "rstq_graph_replay"      I [P])
(defrstq graph-destroy*      "rstq_graph_destroy"     I [P])
(defrstq event-create*       "rstq_event_create"      I [P P I])
(defrstq event-record*       "rstq_event_record"      I [P])
(defrstq event-elapsed-ms*   "rstq_event_elapsed_ms"  I [P P P])
(defrstq event-destroy*      "rstq_event_destroy"     I [P])
(defrstq launch-count*       "rstq_launch_count"      I [P P])
;; ---- decode-chain neighbours
(defrstq rms-norm*           "rstq_rms_norm"            I [P P P P L L D D])       ; ctx x weight out rows features eps gain-offset
(defrstq rms-norm-quant-act* "rstq_rms_norm_quant_act"  I [P P P P P P L L D D])
(defrstq silu-mul*           "rstq_silu_mul"            I [P P P P L])
(defrstq gelu-mul*           "rstq_gelu_mul"            I [P P P P L])
(defrstq residual-add*       "rstq_residual_add"        I [P P P P L])
(defrstq rope-pos*           "rstq_rope_pos"            I [P P P P L L D L])       ; ctx x out posbuf heads head-dim theta pos
(defrstq kv-append*          "rstq_kv_append"           I [P P P P L L L])         ; ctx src cache posbuf kvrow pos maxpos
(defrstq rope-append*        "rstq_rope_append"         I [P P P P P P P L L L D L L])
(defrstq gqa-decode-attention* "rstq_gqa_decode_attention" I [P P P P P P L L L L L L D])
(defrstq gqa-decode-attention-quant-act* "rstq_gqa_decode_attention_quant_act" I [P P P P P P P P P L L L L L L D])
(defrstq residual-rms-norm-quant-act* "rstq_residual_rms_norm_quant_act" I [P P P P P P P P L L D D])
(defrstq silu-mul-quant-act* "rstq_silu_mul_quant_act"  I [P P P P P P L])
(defrstq gelu-mul-quant-act* "rstq_gelu_mul_quant_act"  I [P P P P P P L])
;; ---- sharded weights
(defrstq tp-region-bytes*    "rstq_tp_region_bytes"   L [I L])
(defrstq tp-attach*          "rstq_tp_attach"         I [P P P I I I L])           ; ctx regions tp** dev rank nranks region-bytes
(defrstq tp-create-local*    "rstq_tp_create_local"   I [P P P I L])               ; ctx devs tps nranks max-payload
(defrstq tp-allgather*       "rstq_tp_allgather"      I [P P P L L])
(defrstq tp-allreduce-f32*   "rstq_tp_allreduce_f32"  I [P P P L])
(defrstq tp-qmatmul*         "rstq_tp_qmatmul"        I [P P P P L I I I])         ; tp w x y M act mode split
(defrstq tp-free*            "rstq_tp_free"           I [P])
(defrstq ipc-export*         "rstq_ipc_export"        I [P P])
(defrstq ipc-open*           "rstq_ipc_open"          I [P P P I])                 ; ctx handle64 device-ptr* dev
(defrstq ipc-close*          "rstq_ipc_close"         I [P P I])

;; ---------------------------------------------------------------------------
;; Status wrapper (the shape of cl-call!, ocl_runtime.clj:192-199)
;; ---------------------------------------------------------------------------

(defn- last-error []
  (.getString (.reinterpret ^MemorySegment (.invoke @last-error*) 512) 0))

(defn rstq!
  "Throws ex-info {:function :error :message} unless `rc` is RSTQ_OK."
  [fname rc]
  (when-not (zero? (long rc))
    (throw (ex-info (str fname " failed: " (last-error)) {:function fname :error rc :message (last-error)})))
  rc)

(defmacro ^:private call [h fname & args]
  `(rstq! ~fname (.invokeWithArguments ^java.lang.invoke.MethodHandle @~h (object-array [~@args]))))

;; ---------------------------------------------------------------------------
;; Runtime state: one context over the visible devices, one in-order queue per device
;; (ocl_runtime.clj:205-215 keeps the same in a `state` atom)
;; ---------------------------------------------------------------------------

(defonce ^:private state (atom nil))
(def ^:dynamic *current-arena* nil)                      ; ocl_runtime.clj:222-224

(def dtype-bytes {:float 4 :int 4 :byte 1 :int8 1 :half 2 :bf16 2 :long 8 :double 8})
(def RSTQ_F32 0) (def RSTQ_BF16 1)
(def RSTQ_MODE_F 0) (def RSTQ_MODE_A8 1)

(defn- out-ptr ^MemorySegment [^Arena a] (.allocate a ValueLayout/ADDRESS))
(defn- deref-ptr ^MemorySegment [^MemorySegment s] (.get s ValueLayout/ADDRESS 0))

(defn query-devices
  "[{:id :cuda:N :sm-count :l2-bytes :memory-bytes :compute-capability}] of the devices of the context."
  []
  (when-let [{:keys [ctx ndev]} @state]
    (with-open [a (Arena/ofConfined)]
      (vec (for [d (range ndev)]
             (let [o (.allocate a 32 8)]
               (call device-info* "rstq_device_info" ctx o (int d))
               {:id (keyword (str "cuda:" d))
                :sm-count (.get o ValueLayout/JAVA_LONG 0) :l2-bytes (.get o ValueLayout/JAVA_LONG 8)
                :memory-bytes (.get o ValueLayout/JAVA_LONG 16)
                :compute-capability (.get o ValueLayout/JAVA_LONG 24)}))))))

(defn init!
  "Creates the context over `ordinals` (default: every CUDA device).  Idempotent."
  ([] (init! nil))
  ([ordinals]
   (or @state
       (with-open [a (Arena/ofConfined)]
         (let [n (or (some-> ordinals count)
                     (let [c (.allocate a ValueLayout/JAVA_INT)]
                       (call device-count* "rstq_device_count" c)
                       (.get c ValueLayout/JAVA_INT 0)))
               devs (.allocateFrom a ValueLayout/JAVA_INT (int-array (or ordinals (range n))))
               out (out-ptr a)]
           (call init* "rstq_init" devs out (int n))
           (reset! state {:ctx (deref-ptr out) :ndev n :kernels (atom {})}))))))

(defn shutdown! []
  (when-let [{:keys [ctx]} @state]
    (call shutdown* "rstq_shutdown" ctx)
    (reset! state nil)))

(defn- ctx [] (:ctx (or @state (init!))))

;; ---- kernel arenas (ocl_runtime.clj:533-562): a scope that owns what is made inside it
(defn make-kernel-arena! [] (atom {:buffers [] :prepared [] :graphs []}))
(defn close-kernel-arena! [arena]
  (doseq [g (:graphs @arena)] (call graph-destroy* "rstq_graph_destroy" g))
  (doseq [b (:buffers @arena)] (call free* "rstq_free" (:segment b)))
  (reset! arena {:buffers [] :prepared [] :graphs []}))
(defn- own! [kind v] (when *current-arena* (swap! *current-arena* update kind conj v)) v)

;; ---- buffers (ocl_runtime.clj:405-499): the same record shape {:segment :n-elements :byte-size :dtype}
(defn make-buffer
  ([n dtype] (make-buffer n dtype 0))
  ([n dtype dev]
   (with-open [a (Arena/ofConfined)]
     (let [bytes (* (long n) (long (dtype-bytes dtype))) out (out-ptr a)]
       (call alloc* "rstq_alloc" (ctx) out (int dev) (long (max bytes 1)))
       (own! :buffers {:segment (deref-ptr out) :n-elements n :byte-size bytes :dtype dtype :device dev})))))

(defn free-buffer! [buf] (call free* "rstq_free" (:segment buf)) nil)

(defn array->buffer!
  "Copies a JVM primitive array into `buf` (dtype-switched like ocl_runtime.clj:452-470)."
  [buf arr]
  (let [seg (MemorySegment/ofArray arr)]
    (call upload* "rstq_upload" (:segment buf) seg 0 (.byteSize seg))
    buf))

(defn buffer->array
  "Reads `buf` back into a fresh JVM array of its dtype (:half / :bf16 travel as short[])."
  [buf]
  (let [n (int (:n-elements buf))
        arr (case (:dtype buf)
              :float (float-array n) :int (int-array n) (:byte :int8) (byte-array n)
              (:half :bf16) (short-array n) :long (long-array n) :double (double-array n))]
    (call download* "rstq_download" (:segment buf) (MemorySegment/ofArray arr) 0 (long (:byte-size buf)))
    arr))

(defn buffer-of-array
  "A buffer record over device memory somebody else owns (`address` as this device sees it)."
  [address n dtype dev]
  (with-open [a (Arena/ofConfined)]
    (let [out (out-ptr a) bytes (* (long n) (long (dtype-bytes dtype)))]
      (call buf-wrap* "rstq_buf_wrap" (ctx) out (MemorySegment/ofAddress address) (int dev) bytes)
      {:segment (deref-ptr out) :n-elements n :byte-size bytes :dtype dtype :device dev :external? true})))

(defn buffer-as-float-buffer [buf] (assoc buf :dtype :float :n-elements (quot (:byte-size buf) 4)))
(defn buffer-as-int-buffer   [buf] (assoc buf :dtype :int   :n-elements (quot (:byte-size buf) 4)))

;; ---- registered kernels (ocl_runtime.clj:568-576, 974-1049).  A registered kernel of this runtime is
;; one of the library's operators under the reference's operator name; kernels generated from source
;; (`:map-void` through a run-time compiler) are not part of this path.
(defn register-kernel! [kname f] (swap! (:kernels (or @state (init!))) assoc kname f) kname)
(defn kernel-registry-entry [kname] (get @(:kernels (or @state (init!))) kname))

(defn invoke-registered-map-void-kernel
  "Runs kernel `kname` on `arrays` (buffer records) and `scalars` now."
  [kname arrays scalars n]
  (if-let [f (kernel-registry-entry kname)]
    (apply f (concat arrays scalars [n]))
    (throw (ex-info "kernel not registered" {:kernel-name kname}))))

(defn bind-registered-map-void-kernel
  "Binds a launch once; the handle is launched any number of times (or recorded into a graph)."
  [kname arrays scalars n]
  (when-not (kernel-registry-entry kname) (throw (ex-info "kernel not registered" {:kernel-name kname})))
  (own! :prepared {:bound (fn [] (invoke-registered-map-void-kernel kname arrays scalars n))
                   :group-count 1 :kernel-name kname :async? true}))

(defn launch-registered-bound! [prepared] ((:bound prepared)) prepared)

;; ---- graphs (ocl_runtime.clj:1051-1084)
(defn record-graph!
  "Records the launches `thunk` makes on device `dev` into one replayable graph."
  ([thunk] (record-graph! thunk 0))
  ([thunk dev]
   (with-open [a (Arena/ofConfined)]
     (let [out (out-ptr a)]
       (call graph-begin* "rstq_graph_begin" (ctx) (int dev))
       (try (thunk)
            (finally (call graph-end* "rstq_graph_end" (ctx) out (int dev))))
       (own! :graphs (deref-ptr out))))))
(defn replay-graph! [g] (call graph-replay* "rstq_graph_replay" g) g)
(defn destroy-graph! [g] (call graph-destroy* "rstq_graph_destroy" g) nil)
(defn destroy-prepared! [_prepared] nil)                 ; a bound launch owns nothing native

(defn synchronize-async!
  "Waits for device `dev`; a time-bounded wait that ran out inside a kernel surfaces here (RSTQ_E_WAIT)."
  ([] (synchronize-async! 0))
  ([dev] (call sync* "rstq_sync" (ctx) (int dev)) nil))

;; ---- per-kernel device timing for profile-program! (gpu/core.clj:1343-1388)
(defn timed-launch!
  "Runs `thunk` between two device events on `dev`; returns milliseconds."
  [thunk dev]
  (with-open [a (Arena/ofConfined)]
    (let [e0 (out-ptr a) e1 (out-ptr a) ms (.allocate a ValueLayout/JAVA_FLOAT)]
      (call event-create* "rstq_event_create" (ctx) e0 (int dev))
      (call event-create* "rstq_event_create" (ctx) e1 (int dev))
      (call event-record* "rstq_event_record" (deref-ptr e0))
      (thunk)
      (call event-record* "rstq_event_record" (deref-ptr e1))
      (call event-elapsed-ms* "rstq_event_elapsed_ms" (deref-ptr e0) (deref-ptr e1) ms)
      (call event-destroy* "rstq_event_destroy" (deref-ptr e0))
      (call event-destroy* "rstq_event_destroy" (deref-ptr e1))
      (.get ms ValueLayout/JAVA_FLOAT 0))))
