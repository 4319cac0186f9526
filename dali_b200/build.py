"""Builds libdali_b200.so in-tree (dali_b200/lib/).

Host C++ goes through g++, CUDA sources through nvcc for sm_100a only
(-gencode arch=compute_100a,code=sm_100a).  The device prelude that is spliced
in front of every run-time generated kernel is embedded as a string literal.
Run as `python -m dali_b200.build` or through __graft_entry__.build().
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
LIB = os.path.join(LIBDIR, "libdali_b200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-sign-compare", "-I" + os.path.join(CUDA_HOME, "include"),
             "-I" + os.path.join(HERE, "host", "include")]


def _embed_prelude():
    # the peer-exchange layout and its device helpers come first: generated kernels that reduce across ranks use them
    src = "".join(open(os.path.join(CSRC, f)).read() + "\n" for f in ("peer.h", "peer_device.cuh", "prelude.cuh"))
    assert ')DALIPRELUDE"' not in src
    out = os.path.join(CSRC, "prelude_embed.inc")
    text = 'R"DALIPRELUDE(' + src + ')DALIPRELUDE"\n'
    if not os.path.exists(out) or open(out).read() != text:
        with open(out, "w") as f:
            f.write(text)


def _embed(src_name, out_name, tag):
    src = open(os.path.join(CSRC, src_name)).read()
    close = ")" + tag + '"'
    assert close not in src
    out = os.path.join(CSRC, out_name)
    text = 'R"' + tag + "(" + src + close + "\n"
    if not os.path.exists(out) or open(out).read() != text:
        with open(out, "w") as f:
            f.write(text)


def _embed_source_hash():
    """A hash of everything that decides what a generated kernel looks like and how its parameter block is laid out:
    part of every cache key, so that a cubin written by another build of the library is never loaded by this one."""
    import hashlib
    h = hashlib.sha256()
    for f in ("codegen.cc", "codegen.h", "plan.cc", "ir.cc", "ir.h", "gemm_sm100.cc", "gemm_sm100.cuh", "peer.h", "peer_device.cuh",
              "prelude.cuh"):
        h.update(open(os.path.join(CSRC, f), "rb").read())
    out = os.path.join(CSRC, "source_hash.inc")
    text = '"' + h.hexdigest()[:16] + '"\n'
    if not os.path.exists(out) or open(out).read() != text:
        with open(out, "w") as f:
            f.write(text)


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd, log=None):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log:
        with open(log, "w") as f:
            f.write(" ".join(cmd) + "\n" + r.stdout)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("build step failed: " + " ".join(cmd))
    return r.stdout


def build(force=False, verbose=False):
    os.makedirs(LIBDIR, exist_ok=True)
    objdir = os.path.join(LIBDIR, "obj")
    os.makedirs(objdir, exist_ok=True)
    _embed_prelude()
    _embed("gemm_sm100.cuh", "gemm_embed.inc", "DALIGEMM")
    _embed_source_hash()
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh", ".inc"))]
    headers += [os.path.join(HERE, "..", "include", f) for f in os.listdir(os.path.join(HERE, "..", "include"))]
    for root, _, files in os.walk(os.path.join(HERE, "host", "include")):
        headers += [os.path.join(root, f) for f in files if f.endswith(".h")]
    objs = []
    srcs = []
    for root, _, files in os.walk(CSRC):
        for f in sorted(files):
            if f.endswith((".cc", ".cu")):
                srcs.append(os.path.join(root, f))
    for src in srcs:
        obj = os.path.join(objdir, os.path.relpath(src, CSRC).replace(os.sep, "_") + ".o")
        objs.append(obj)
        if not force and not _newer(obj, [src] + headers):
            continue
        if src.endswith(".cu"):
            cmd = [os.path.join(CUDA_HOME, "bin", "nvcc")] + NVCC_FLAGS + ["-I" + CSRC, "-c", src, "-o", obj]
            out = _run(cmd, log=obj + ".ptxas.log")   # registers / spills / shared memory per kernel
            if verbose:
                print(out)
        else:
            _run(["g++"] + CXX_FLAGS + ["-I" + CSRC, "-c", src, "-o", obj])
    if force or _newer(LIB, objs):
        libdir = os.path.join(CUDA_HOME, "lib64")
        _run(["g++", "-shared", "-o", LIB] + objs +
             ["-L" + libdir, "-lcudart_static", "-lnvrtc", "-ldl", "-lrt", "-lpthread",
              "-Wl,-rpath," + libdir, "-Wl,--no-undefined"])
    return LIB


def build_program(source, output):
    """Compiles a C++ program written against the front end's headers (dali/array/array.h, op.h) and links it
    with the library; the library is found next to the program at run time."""
    lib = build()
    inc = os.path.join(HERE, "host", "include")
    if _newer(output, [source, lib]):
        _run(["g++", "-std=c++14", "-O1", "-I" + inc, "-I" + os.path.join(HERE, "..", "include"), source, "-o", output,
              "-L" + LIBDIR, "-ldali_b200",
              "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + LIBDIR])
    return output


def build_programs():
    """The C++ programs of the package (dali_b200/host/programs): built next to the library."""
    out = []
    pdir = os.path.join(HERE, "host", "programs")
    for f in sorted(os.listdir(pdir)):
        if f.endswith(".cpp"):
            out.append(build_program(os.path.join(pdir, f), os.path.join(LIBDIR, f[:-4])))
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
