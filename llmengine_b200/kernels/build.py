"""Compiling the CUDA sources of `csrc/` for sm_100a into shared libraries, one
per source file, inside the package folder.

Each library is built the first time something needs it, so a run compiles only
what its model and dtype use; `build_all()` compiles everything (used by the
"does it build" check, which needs no GPU because nvcc cross-compiles).  A
library's file name carries a hash of its source, the shared header and the
flags, so a changed source never loads a stale binary.  While nvcc runs, a line
is printed every few seconds.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import Dict, Iterable, List, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(_HERE), "csrc")

# library name -> source file
SOURCES: Dict[str, str] = {
    "elementwise": "elementwise.cu",
    "attention_plain": "attention_plain.cu",
    "gemm_f32": "gemm_f32.cu",
    "sampling": "sampling.cu",
    "gemm_skinny": "gemm_skinny.cu",
    "gemm_tcgen05": "gemm_tcgen05.cu",
    "utility": "utility.cu",
    # the step executor (host code): walks a model's plan and launches the kernels of the other libraries
    "executor": "executor.cu",
    # the engine as a C++ library (include/llmengine_b200/engine.h): native host code over the executor and the kernels
    "engine": "native/engine.cu",
    # compiled per head size: ask for "attention_fast@HEAD_DIM=128"
    "attention_fast": "attention_fast.cu",
    # the tcgen05 portion kernel, per head size (64 or 128): "attention_tc@HEAD_DIM=128"
    "attention_tc": "attention_tc.cu",
    # the same kernels with built-in scratch memory: "attention_decode_static@HEAD_DIM=128"
    "attention_decode_static": "attention_decode_static.cu",
}

# sources that a library's source file includes (they count for its hash)
INCLUDES: Dict[str, List[str]] = {"attention_decode_static": ["attention_fast.cu"]}

# libraries that need compile-time values, and the values `build_all` compiles them for
VARIANTS: Dict[str, List[str]] = {
    "attention_fast": ["attention_fast@HEAD_DIM=64", "attention_fast@HEAD_DIM=128"],
    "attention_decode_static": ["attention_decode_static@HEAD_DIM=128"],
    "attention_tc": ["attention_tc@HEAD_DIM=64", "attention_tc@HEAD_DIM=128"],
}

INCLUDE = os.path.join(os.path.dirname(_HERE), "include")

# link flags of single libraries
LINK: Dict[str, List[str]] = {"executor": ["-ldl"], "engine": ["-ldl"]}

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[llmengine_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("LLMENGINE_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc was not found (looked at $LLMENGINE_NVCC, PATH and /usr/local/cuda/bin); "
                     "the kernels of this engine have to be compiled for sm_100a")


def build_dir() -> str:
    """`<package>/_build` when it can be written, else a per-user folder under the temp dir."""
    d = os.path.join(os.path.dirname(_HERE), "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"llmengine_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def split_key(key: str):
    """"name@A=1,B=2" -> ("name", ["-DA=1", "-DB=2"])."""
    name, _, rest = key.partition("@")
    if name not in SOURCES:
        raise BuildError(f"no kernel library named {name!r}; known: {', '.join(sorted(SOURCES))}")
    defines = [f"-D{d}" for d in rest.split(",") if d]
    if name in VARIANTS and not defines:
        raise BuildError(f"library {name!r} needs compile-time values, e.g. {VARIANTS[name][0]!r}")
    return name, defines


def _digest(key: str) -> str:
    name, defines = split_key(key)
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + defines).encode())
    for fn in sorted(os.listdir(CSRC)):
        if (fn.endswith((".cuh", ".h")) or fn == SOURCES[name] or fn in INCLUDES.get(name, ())) and os.path.isfile(os.path.join(CSRC, fn)):
            with open(os.path.join(CSRC, fn), "rb") as f:
                h.update(fn.encode())
                h.update(f.read())
    if os.path.dirname(SOURCES[name]):                      # a source in a folder of its own: its neighbours count
        sub = os.path.join(CSRC, os.path.dirname(SOURCES[name]))
        for fn in sorted(os.listdir(sub)):
            with open(os.path.join(sub, fn), "rb") as f:
                h.update(fn.encode())
                h.update(f.read())
    if name in ("executor", "engine"):                      # the libraries behind the public headers
        for root, _dirs, files in sorted(os.walk(INCLUDE)):
            for fn in sorted(files):
                with open(os.path.join(root, fn), "rb") as f:
                    h.update(fn.encode())
                    h.update(f.read())
    return h.hexdigest()[:12]


def library_path(key: str) -> str:
    name, defines = split_key(key)
    tag = "".join("_" + d[2:].replace("=", "") for d in defines)
    return os.path.join(build_dir(), f"llme_{name}{tag}_{_digest(key)}.so")


def ensure_built(names: Iterable[str], extra_flags: Optional[List[str]] = None) -> Dict[str, str]:
    """Compile the named libraries that are not built yet (in parallel) and return their paths."""
    names = list(dict.fromkeys(names))
    paths = {n: library_path(n) for n in names}
    todo = [n for n in names if not os.path.exists(paths[n])]
    if not todo:
        if _manifest_differs(paths):       # a source went back to a state whose library was still there
            write_manifest(names)
        return paths
    nvcc = find_nvcc()
    procs = {}
    t0 = time.time()
    for n in todo:
        tmp = f"{paths[n]}.{os.getpid()}.tmp"
        name, defines = split_key(n)
        cmd = [nvcc, *NVCC_FLAGS, *defines, *(extra_flags or []), "-I", CSRC, "-I", INCLUDE, "-o", tmp,
               os.path.join(CSRC, SOURCES[name]), *LINK.get(name, [])]
        _log(f"compiling {SOURCES[name]} {' '.join(defines)} for sm_100a ...".replace("  ", " "))
        log = tempfile.TemporaryFile(mode="w+")          # not a pipe: a long error listing must not block nvcc
        procs[n] = (subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT, text=True), tmp, log)
    last = time.time()
    pending = dict(procs)
    while pending:
        for n, (p, tmp, log) in list(pending.items()):
            if p.poll() is None:
                continue
            log.seek(0)
            out = log.read()
            log.close()
            del pending[n]
            if p.returncode != 0:
                for _, (q, _qtmp, _qlog) in pending.items():
                    q.kill()
                raise BuildError(f"nvcc failed on {n} (exit {p.returncode}):\n{out}")
            os.replace(tmp, paths[n])
            _log(f"built {os.path.basename(paths[n])} in {time.time() - t0:.0f} s")
        if pending:
            time.sleep(0.2)
            if time.time() - last > 8:
                last = time.time()
                _log(f"still compiling {', '.join(sorted(pending))} ({last - t0:.0f} s)")
    write_manifest(names)
    return paths


def all_keys() -> List[str]:
    keys = [n for n in SOURCES if n not in VARIANTS]
    for v in VARIANTS.values():
        keys.extend(v)
    return keys


def _manifest_differs(paths: Dict[str, str]) -> bool:
    import json
    try:
        with open(os.path.join(build_dir(), "manifest.json"), "r", encoding="utf-8") as f:
            known = json.load(f)
    except (OSError, ValueError):
        return True
    return any(known.get(k) != os.path.basename(p) for k, p in paths.items())


def write_manifest(more: Iterable[str] = ()) -> str:
    """`manifest.json` in the build folder: library key -> file name, for every library that is built.  The C++
    front (include/llmengine_b200/engine.h) finds the kernel libraries through it."""
    import json
    d = build_dir()
    path = os.path.join(d, "manifest.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            known = json.load(f)
    except (OSError, ValueError):
        known = {}
    for key in list(all_keys()) + list(more):
        p = library_path(key)
        if os.path.exists(p):
            known[key] = os.path.basename(p)
    known = {k: v for k, v in known.items() if os.path.exists(os.path.join(d, v))}
    tmp = f"{path}.{os.getpid()}.tmp"
    with open(tmp, "w", encoding="utf-8") as f:
        json.dump(known, f, indent=1, sort_keys=True)
    os.replace(tmp, path)
    if "engine" in known:                 # a fixed name to link a C++ program against (-lllmengine_b200)
        link = os.path.join(d, "libllmengine_b200.so")
        try:
            if os.path.islink(link) or os.path.exists(link):
                os.unlink(link)
            os.symlink(known["engine"], link)
        except OSError:
            pass
    return path


def build_all() -> Dict[str, str]:
    paths = ensure_built(all_keys())
    write_manifest()
    return paths


if __name__ == "__main__":
    # python -m llmengine_b200.kernels.build [library keys ...]: compile them (all of them without arguments)
    import sys as _sys
    built = ensure_built(_sys.argv[1:]) if len(_sys.argv) > 1 else build_all()
    write_manifest(built)
    for k, v in built.items():
        print(f"{k}: {v}")
