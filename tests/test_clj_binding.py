"""The Clojure binding files against include/rstq.h.

clj/raster/gpu/cuda_runtime.clj declares every native function once, as
`(defrstq var "c_symbol" RET [ARG ...])` with one-letter Panama layouts (I int32, L int64, F float,
D double, P address).  No JVM exists where this repository is tested, so the binding cannot run; what
can be pinned is that each declared descriptor is the C prototype: same symbol, same arity, the same
pointer / scalar kind in the same order, the same return kind.  The header's own rule -- pointers
first, then scalars, the convention of the reference's generated C kernels
(src/raster/compiler/backend/cpu/aot.clj:428-434) -- and the ctypes table of raster_b200/_lib.py are
checked the same way.  CPU only.
"""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_prototypes():
    src = open(os.path.join(ROOT, "include", "rstq.h")).read()
    src = re.sub(r"/\*.*?\*/", " ", src, flags=re.S)
    protos = {}
    for m in re.finditer(r"RSTQ_API\s+([^;(]+?)\s*(\brstq_\w+)\s*\(([^;]*?)\)\s*;", src, flags=re.S):
        ret, name, params = m.group(1).strip(), m.group(2), re.sub(r"\s+", " ", m.group(3)).strip()
        kinds = []
        if params and params != "void":
            for p in params.split(","):
                p = p.strip()
                if "*" in p:
                    kinds.append("P")
                elif re.search(r"\bint32_t\b", p):
                    kinds.append("I")
                elif re.search(r"\bint64_t\b", p):
                    kinds.append("L")
                elif re.search(r"\bdouble\b", p):
                    kinds.append("D")
                elif re.search(r"\bfloat\b", p):
                    kinds.append("F")
                else:
                    raise AssertionError(f"{name}: parameter type not a C scalar or pointer: {p}")
        rk = "P" if "*" in ret else "L" if "int64_t" in ret else "I"
        protos[name] = (rk, kinds)
    return protos


def clj_descriptors():
    src = open(os.path.join(ROOT, "clj", "raster", "gpu", "cuda_runtime.clj")).read()
    out = {}
    for m in re.finditer(r'\(defrstq\s+([^\s]+)\s+"(rstq_\w+)"\s+([ILFDP])\s+\[([ILFDP\s]*)\]\)', src):
        assert m.group(2) not in out, f"{m.group(2)} declared twice"
        out[m.group(2)] = (m.group(1), m.group(3), m.group(4).split())
    return out


def test_every_exported_function_is_declared_once_with_the_prototype_of_the_header():
    protos, descs = header_prototypes(), clj_descriptors()
    assert len(protos) >= 70
    assert sorted(descs) == sorted(protos), (sorted(set(protos) - set(descs)), sorted(set(descs) - set(protos)))
    for name, (ret, kinds) in protos.items():
        var, cret, ckinds = descs[name]
        assert cret == ret, f"{name}: returns {ret}, bound as {cret}"
        assert ckinds == kinds, f"{name}: prototype {kinds}, bound as {ckinds}"


def test_pointers_come_first_then_scalars_in_every_signature():
    for name, (_, kinds) in header_prototypes().items():
        seen_scalar = False
        for k in kinds:
            if k == "P":
                assert not seen_scalar, f"{name}: a pointer follows a scalar ({kinds})"
            else:
                seen_scalar = True


def test_ctypes_table_matches_the_header_too():
    from raster_b200 import _lib as L
    kind = {C.c_int32: "I", C.c_int64: "L", C.c_double: "D", C.c_float: "F"}
    protos = header_prototypes()
    assert sorted(L.SIGNATURES) == sorted(protos)
    for name, args in L.SIGNATURES.items():
        got = [kind.get(a, "P") for a in args]
        assert got == protos[name][1], f"{name}: header {protos[name][1]}, ctypes {got}"


def test_cuda_methods_keep_the_reference_arities_and_register_their_facets():
    src = open(os.path.join(ROOT, "clj", "raster", "quant", "cuda.clj")).read()
    # (name, number of typed parameters) as in src/raster/quant/op.clj:43-99, train.clj:88-89, 110-113,
    # kernels_k.clj:349-351
    want = {"raster.quant.op/qlinear-i8!": 6, "raster.quant.op/qlinear-i8": 5,
            "raster.quant.op/qlinear-i8-q8!": 6, "raster.quant.op/qlinear-i8-q8": 5,
            "raster.quant.train/qlinear-q8": 6, "raster.quant.train/qlinear-q8-dx": 6,
            "raster.quant.kernels-k/qmatmul-i8-gemm!": 8}
    for name, arity in want.items():
        m = re.search(r"\(deftm\s+(?:\^:no-inline\s+)?" + re.escape(name) + r"\s+(?:\"[^\"]*\"\s+)?\[(.*?)\]\s*:-", src, flags=re.S)
        assert m, f"no CUDA method for {name}"
        assert len(re.findall(r":-", m.group(1))) == arity, f"{name}: arity"
    for form in ("register-buffer-write! 'raster.quant.op/qlinear-i8!    :overwrite 3",
                 "register-buffer-write! 'raster.quant.op/qlinear-i8-q8! :overwrite 3",
                 "register-placement! op :gpu-quant"):
        assert form in src
    # every handle the methods use exists in the runtime table
    descs = {v[0] for v in clj_descriptors().values()}
    for used in re.findall(r"@#'rt/([\w\-\*]+)", src):
        assert used in descs, f"cuda.clj uses rt/{used}, not declared in cuda_runtime.clj"
