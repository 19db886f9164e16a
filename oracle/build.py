#!/usr/bin/env python3
"""Build the checker artefacts.  TEST INFRASTRUCTURE ONLY -- nothing in the product
package imports this file or anything it builds.

  oracle/liblt_oracle.so        the CPU restatement (lt_oracle.c), gcc, OpenMP
  oracle/_ref/libbpd_cpu.so     the reference's own CPU Q8_0 library, compiled from its
                                sources where they lie in the reference checkout
  oracle/_ref/*.cubin           the reference's own CUDA kernel texts (the string
                                constants of its resident engine and the text its
                                Prolog emitters print), compiled for sm_100a

The `_ref` outputs exist only where a reference checkout is present (pass its root
with --reference or the LLAMATOV_REFERENCE environment variable); they are binaries,
never sources, and are git-ignored.  A box without the checkout uses the prebuilt
files that travelled with the tree.
"""
import argparse
import ast
import os
import re
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
REF_OUT = os.path.join(HERE, "_ref")
ORACLE_SO = os.path.join(HERE, "liblt_oracle.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _run(cmd, **kw):
    r = subprocess.run(cmd, capture_output=True, text=True, **kw)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout[-2000:], r.stderr[-4000:]))
    return r


def _stale(out, srcs):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(s) > t for s in srcs)


def build_oracle(force=False):
    src = os.path.join(HERE, "lt_oracle.c")
    if force or _stale(ORACLE_SO, [src, __file__]):
        # -ffp-contract=off: the only fused multiply-adds are the explicit fmaf() calls.
        # -mfma lets fmaf() be one instruction (same single rounding as libm's fmaf).
        _run(["gcc", "-O3", "-ffp-contract=off", "-mfma", "-mavx2", "-fopenmp", "-shared", "-fPIC",
              "-o", ORACLE_SO, src, "-lm"])
    return ORACLE_SO


# --------------------------------------------------------------------------- _ref

def _python_string_constants(path, names):
    """String constants assigned at module level in a Python file, read with `ast`
    (the file is parsed, never executed)."""
    tree = ast.parse(open(path, encoding="utf-8").read())
    out = {}
    for node in tree.body:
        if isinstance(node, ast.Assign) and len(node.targets) == 1 and isinstance(node.targets[0], ast.Name):
            n = node.targets[0].id
            if n in names and isinstance(node.value, ast.Constant) and isinstance(node.value.value, str):
                out[n] = node.value.value
    missing = set(names) - set(out)
    if missing:
        raise RuntimeError("constants not found in %s: %s" % (path, sorted(missing)))
    return out


_FMT = re.compile(r'format\(S,\s*"((?:[^"\\]|\\.)*)",\s*\[([^\]]*)\]\)')


def _render_prolog_clause(path, head, bindings):
    """Print what one `emit_*` clause of a Prolog emitter prints: the clause is a list of
    format(S, "text", [Args]) goals; ~w takes the next argument, ~n is a newline.  Only the
    directives those clauses use are handled.  `bindings` maps Prolog variable names to text."""
    text = open(path, encoding="utf-8").read()
    start = text.index(head)
    end = text.index("close(S)", start)
    out = []
    for m in _FMT.finditer(text[start:end]):
        fmt, args = m.group(1), [a.strip() for a in m.group(2).split(",") if a.strip()]
        fmt = fmt.replace('\\"', '"').replace("\\\\", "\\")
        it = iter(args)

        def sub(mm):
            if mm.group(0) == "~n":
                return "\n"
            a = next(it)
            return str(bindings[a])
        out.append(re.sub(r"~w|~n", sub, fmt))
    return "".join(out)


def reference_kernel_sources(ref_root):
    """name -> CUDA text of each reference kernel on the decode path."""
    dr = os.path.join(ref_root, "bpd", "lib", "dev_residency.py")
    emit = os.path.join(ref_root, "bpd", "kernelgen", "emitters")
    consts = _python_string_constants(dr, [
        "_QUANT_SRC_PAR", "_QUANT_SRC", "_SILU_QUANT_SRC", "_ATTN_DECODE_MASKED_SRC_TMPL",
        "_ARGMAX2_SRC", "_ARGMAX_SRC", "_APPEND_AT_LEN_SRC", "_ADD_SRC", "_SILU_MUL_SRC"])
    src = {
        "quant_q8_par": consts["_QUANT_SRC_PAR"],
        "quant_q8_serial": consts["_QUANT_SRC"],
        "silu_mul_quant": consts["_SILU_QUANT_SRC"],
        "argmax2": consts["_ARGMAX2_SRC"],
        "argmax": consts["_ARGMAX_SRC"],
        "append_at_len": consts["_APPEND_AT_LEN_SRC"],
        "add": consts["_ADD_SRC"],
        "silu_mul": consts["_SILU_MUL_SRC"],
    }
    for maxt in (256, 512):
        src["attn_decode_masked_%d" % maxt] = consts["_ATTN_DECODE_MASKED_SRC_TMPL"] % {"MAXT": maxt}
    # the banked split-order attention: a %-template in the reference's experimental directory
    split = os.path.join(ref_root, "bpd", "kernelgen", "experimental", "attn_decode_split.cu")
    if os.path.exists(split):
        text = open(split).read()
        for ns in (2, 4):
            src["attn_decode_split_%d" % ns] = text % {"MAXT": 256, "NSPLIT": ns}
    hdr = "#include <cuda_fp16.h>\n"
    q8 = os.path.join(emit, "q8_0_from_facts.pl")
    b = {"BM": 16, "BK": 256, "BlockSz": 512}
    src["q8_gemv_tiled_v4"] = hdr + _render_prolog_clause(q8, "emit_q8_0_gemv_tiled_v4(BM, BK, OutFile) :-", b)
    src["q8_gemv_tiled_v4_addres"] = hdr + _render_prolog_clause(
        q8, "emit_q8_0_gemv_tiled_v4_addres(BM, BK, OutFile) :-", b)
    src["q8_gemv_canonical_serial"] = hdr + _render_prolog_clause(
        q8, "emit_q8_0_gemv_canonical_serial(OutFile) :-", {"BlockSz": 64})
    ns = os.path.join(emit, "norm_softmax_from_facts.pl")
    for tag, eps in (("1e-06", "1.0e-6"), ("1e-05", "1.0e-5")):
        src["rmsnorm_blockrow_" + tag] = _render_prolog_clause(
            ns, "emit_rmsnorm_cuda_blockrow(Eps, OutFile) :-", {"Eps": eps})
        src["rmsnorm_canonical_serial_" + tag] = _render_prolog_clause(
            ns, "emit_rmsnorm_cuda_canonical_serial(Eps, OutFile) :-", {"Eps": eps})
    rp = os.path.join(emit, "rope_from_facts.pl")
    for tag, theta in (("1e6", "1000000.0"), ("5e5", "500000.0"), ("1e4", "10000.0")):
        src["rope_" + tag] = _render_prolog_clause(rp, "emit_rope_cuda(Theta, OutFile) :-", {"Theta": theta})
    return src


def build_ref(ref_root, force=False):
    """Compile the reference's own code for this box.  Outputs only into oracle/_ref/."""
    os.makedirs(REF_OUT, exist_ok=True)
    built = []
    # (1) the reference's CPU Q8_0 library.  Flags: the sources use F16C and AVX intrinsics
    # without guards; no -mfma / -march=native (the code mirrors a no-FMA machine and
    # contraction would change bits).
    bench = os.path.join(ref_root, "bpd-substrate", "bench")
    cpu_srcs = [os.path.join(bench, "bpd_cpu.c"), os.path.join(bench, "bpd_gemm_q8_0_cpu.c")]
    so = os.path.join(REF_OUT, "libbpd_cpu.so")
    if force or _stale(so, cpu_srcs):
        _run(["gcc", "-O2", "-mavx", "-mf16c", "-shared", "-fPIC", "-w", "-o", so] + cpu_srcs + ["-lm"])
    built.append(so)
    # (2) the reference's CUDA kernels, same flags as its own build line apart from the arch.
    srcs = reference_kernel_sources(ref_root)
    with tempfile.TemporaryDirectory() as tmp:
        for name, text in sorted(srcs.items()):
            out = os.path.join(REF_OUT, name + ".cubin")
            if not force and os.path.exists(out):
                built.append(out)
                continue
            cu = os.path.join(tmp, name + ".cu")
            with open(cu, "w") as f:
                f.write(text)
            _run([NVCC] + ARCH_FLAGS + ["-cubin", "-O3", cu, "-o", out])
            built.append(out)
    return built


def default_reference_root():
    # the LLAMATOV_REFERENCE variable, else a checkout named "reference" beside this repository
    sibling = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference"))
    for cand in (os.environ.get("LLAMATOV_REFERENCE"), sibling):
        if cand and os.path.isdir(os.path.join(cand, "bpd", "lib")):
            return cand
    return None


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--dump-ref-sources", default=None, help="write the rendered kernel texts to a directory (inspection only)")
    a = ap.parse_args(argv)
    print(build_oracle(a.force))
    ref = a.reference or default_reference_root()
    if ref:
        if a.dump_ref_sources:
            os.makedirs(a.dump_ref_sources, exist_ok=True)
            for n, t in reference_kernel_sources(ref).items():
                open(os.path.join(a.dump_ref_sources, n + ".cu"), "w").write(t)
        for p in build_ref(ref, a.force):
            print(p)
    else:
        print("no reference checkout: oracle/_ref not rebuilt", file=sys.stderr)


if __name__ == "__main__":
    main()
