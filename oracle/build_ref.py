"""Builds oracle/_ref/: the reference's own hand-written C tiles, compiled as they stand.

Test infrastructure, not the product.  The reference is Clojure that generates its
native code at run time, but three functions on the quantized-matmul path exist
in it as literal C text, registered as `:c-helper` overrides for the CPU backend
(src/raster/quant/kernels.clj):

    wi8-dot-q4      :97-109    one Q4_0 block dot (maddubs + madd)
    wi8-dot-q4-x8   :116-138   the 8-column Q4_0 tile (dpbusd cascade)
    wi8-dot-q8-x8   :282-302   the 8-column Q8_0 tile (dpbusd cascade)

This script reads that text out of the reference checkout AT BUILD TIME (nothing
of it is stored in this repository), gives each helper the C name the backend
would give it, appends a three-line exported wrapper per helper, and compiles
the file once per instruction-set variant the `#if` cascade inside the helpers
distinguishes:

    libref_avx2.so        -mavx2                      -> maddubs + madd fallback
    libref_avxvnni.so     -mavx2 -mavxvnni            -> vpdpbusd (AVX-VNNI)
    libref_avx512vnni.so  -mavx2 -mavx512vnni -mavx512vl -> vpdpbusd (AVX-512)

The reference compiles with -march=native (src/raster/compiler/backend/cpu/codegen.clj:68-92),
so which branch it takes depends on the host; tests run the variants the host CPU
supports and compare the scalar restatement in rstq_oracle.c with them bit for bit.

Usage: python oracle/build_ref.py [--reference DIR] [--force]
"""
from __future__ import annotations

import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
REFERENCE = os.environ.get("RASTER_REFERENCE", "/root/reference")
KERNELS_CLJ = "src/raster/quant/kernels.clj"

HELPERS = ("wi8-dot-q4", "wi8-dot-q4-x8", "wi8-dot-q8-x8")
VARIANTS = {
    "avx2": ["-mavx2"],
    "avxvnni": ["-mavx2", "-mavxvnni"],
    "avx512vnni": ["-mavx2", "-mavx512vnni", "-mavx512vl"],
}
# CPU flags (as /proc/cpuinfo spells them) a variant needs to RUN
NEEDS = {"avx2": {"avx2"}, "avxvnni": {"avx2", "avx_vnni"},
         "avx512vnni": {"avx2", "avx512_vnni", "avx512vl"}}


def reference_present(root: str = REFERENCE) -> bool:
    return os.path.exists(os.path.join(root, KERNELS_CLJ))


def _read_string(src: str, i: int):
    """Reads one Clojure string literal that starts at src[i] == '"'; returns (value, next index)."""
    assert src[i] == '"'
    out = []
    i += 1
    esc = {"n": "\n", "t": "\t", "\\": "\\", '"': '"', "r": "\r"}
    while src[i] != '"':
        if src[i] == "\\":
            out.append(esc[src[i + 1]])
            i += 2
        else:
            out.append(src[i])
            i += 1
    return "".join(out), i + 1


def _balanced(src: str, i: int) -> int:
    """Index just past the form that opens at src[i] (a paren), skipping strings and ; comments."""
    depth = 0
    while True:
        c = src[i]
        if c == '"':
            _, i = _read_string(src, i)
            continue
        if c == ";":
            i = src.index("\n", i)
            continue
        if c in "([{":
            depth += 1
        elif c in ")]}":
            depth -= 1
            if depth == 0:
                return i + 1
        i += 1


def extract_helper(src: str, name: str):
    """(includes, generator) of the helper registered for raster.quant.kernels/<name>:
    generator(c_name) returns the C text `(str ... c-name ...)` builds."""
    m = re.search(r"\(descriptor/register-c-helper!\s+'raster\.quant\.kernels/" + re.escape(name) + r"\s", src)
    if not m:
        raise RuntimeError(f"no :c-helper registered for {name}")
    form = src[m.start():_balanced(src, m.start())]
    inc = re.search(r":includes\s+\"", form)
    includes, _ = _read_string(form, inc.end() - 1)
    g = re.search(r":gen\s+\(fn\s+\[c-name\]\s+\(str", form)
    if not g:
        raise RuntimeError(f"{name}: :gen is not (fn [c-name] (str ...))")
    start = form.index("(str", g.start())
    body = form[start + 4:_balanced(form, start) - 1]
    parts, i = [], 0
    while i < len(body):
        c = body[i]
        if c == '"':
            s, i = _read_string(body, i)
            parts.append(("lit", s))
        elif body.startswith("c-name", i):
            parts.append(("name", None))
            i += 6
        elif c.isspace():
            i += 1
        else:
            raise RuntimeError(f"{name}: unexpected token in (str ...) at {body[i:i + 20]!r}")

    def gen(c_name: str) -> str:
        return "".join(c_name if k == "name" else s for k, s in parts)
    return includes, gen


def c_source(root: str = REFERENCE) -> str:
    src = open(os.path.join(root, KERNELS_CLJ)).read()
    includes, bodies = [], []
    for name in HELPERS:
        inc, gen = extract_helper(src, name)
        if inc not in includes:
            includes.append(inc)
        bodies.append(gen("raster_quant_kernels_" + name.replace("-", "_")))
    wrappers = """
#define REF_API __attribute__((visibility("default")))
REF_API long ref_wi8_dot_q4(const signed char* wq, long woff, const signed char* xq, long xoff) {
  return raster_quant_kernels_wi8_dot_q4(wq, woff, xq, xoff);
}
REF_API void ref_wi8_dot_q4_x8(const signed char* wqi, long woff, const signed char* xq, long xoff, int* out) {
  raster_quant_kernels_wi8_dot_q4_x8(wqi, woff, xq, xoff, out);
}
REF_API void ref_wi8_dot_q8_x8(const signed char* wqi, long woff, const signed char* xq, long xoff, int* out) {
  raster_quant_kernels_wi8_dot_q8_x8(wqi, woff, xq, xoff, out);
}
REF_API int ref_uses_dpbusd(void) {
#if (defined(__AVX512VNNI__) && defined(__AVX512VL__)) || defined(__AVXVNNI__)
  return 1;
#else
  return 0;
#endif
}
"""
    return "".join(includes) + "\n" + "\n".join(bodies) + wrappers


def cpu_flags() -> set:
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("flags"):
                return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def runnable_variants():
    """Variants whose library exists and whose instructions this CPU has."""
    have = cpu_flags()
    return [v for v in VARIANTS if NEEDS[v] <= have and os.path.exists(lib_path(v))]


def lib_path(variant: str) -> str:
    return os.path.join(OUT, f"libref_{variant}.so")


def build(root: str = REFERENCE, force: bool = False):
    """Writes _ref/ref_helpers.c from the reference checkout and compiles every variant gcc accepts.
    Returns the list of libraries built (or already present)."""
    if not reference_present(root):
        raise RuntimeError(f"reference checkout not found at {root}")
    os.makedirs(OUT, exist_ok=True)
    csrc = os.path.join(OUT, "ref_helpers.c")
    text = c_source(root)
    if force or not os.path.exists(csrc) or open(csrc).read() != text:
        open(csrc, "w").write(text)
        force = True
    built = []
    for variant, flags in VARIANTS.items():
        so = lib_path(variant)
        if force or not os.path.exists(so):
            r = subprocess.run([os.environ.get("CC", "gcc"), "-O2", *flags, "-fvisibility=hidden", "-shared", "-fPIC",
                                "-o", so, csrc], capture_output=True, text=True)
            if r.returncode != 0:      # an older gcc without -mavxvnni: that variant is simply absent
                print(f"[build_ref] {variant}: {r.stderr.strip().splitlines()[-1] if r.stderr else 'failed'}",
                      file=sys.stderr)
                continue
        built.append(so)
    return built


if __name__ == "__main__":
    root = REFERENCE
    if "--reference" in sys.argv:
        root = sys.argv[sys.argv.index("--reference") + 1]
    for p in build(root, force="--force" in sys.argv):
        print(p)
