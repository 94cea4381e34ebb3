"""Builds libasd_b200.so (sm_100a only) in-tree with nvcc.  No torch, no cmake.

The library is made of components; ``build()`` links all of them, ``build(components=("mezilix",))`` only what one
model family needs (a first call on a fresh checkout then compiles nothing else).  Which components the library on
disk holds is recorded beside it; asking for more recompiles the missing objects and links again."""
from __future__ import annotations

import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libasd_b200.so")
MANIFEST = os.path.join(HERE, "build", "components.json")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
         "-Xptxas", "-v", "-DASD_BUILDING_DSO"]

# component -> translation units; "core" is part of every library
COMPONENTS = {
    "core": ["core.cu"],
    "linear": ["gemm.cu", "gemm_tc.cu"],
    "blocks": ["linear_simt.cu", "linear_tc.cu"],
    "latent": ["latent_attention.cu"],
    "rows": ["norm_ops.cu", "moe.cu"],          # row kernels and the expert router that several families share
    "mezilix": ["mezilix_engine.cu", "stream_ops.cu"],
    "rivetar": ["rivetar_engine.cu", "gla.cu", "window_attention.cu"],
    "mavipel": ["mavipel_engine.cu", "delta_rule.cu", "talking_attention.cu"],
    "lukopel": ["lukopel_engine.cu", "residual_streams.cu", "mixed_attention.cu", "mixed_attention_tc.cu"],
    "qwen": ["engine.cu", "layers.cu", "attention.cu", "attention_tc.cu", "forward_persist.cu"],
    "sampling": ["api.cu", "sampler.cu", "stop_rule.cu"],
}
REQUIRES = {"mezilix": ("linear", "blocks", "latent", "rows"), "rivetar": ("linear", "blocks", "latent", "rows"),
            "mavipel": ("linear", "blocks", "rows"), "lukopel": ("linear", "blocks", "rows"), "qwen": ("linear",)}


def all_components():
    return tuple(COMPONENTS)


def _closure(components):
    want = {"core"}
    for c in components:
        if c not in COMPONENTS:
            raise KeyError(f"unknown component {c!r}; have {sorted(COMPONENTS)}")
        want.add(c)
        want.update(REQUIRES.get(c, ()))
    return tuple(c for c in COMPONENTS if c in want)


def sources(components=None):
    comps = _closure(components if components is not None else all_components())
    listed = {f for fs in COMPONENTS.values() for f in fs}
    extra = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu") and f not in listed)
    if extra:
        raise RuntimeError(f"csrc/{extra[0]} belongs to no component of build.py")
    return [os.path.join(CSRC, f) for c in comps for f in COMPONENTS[c]]


def built_components():
    """components of the library on disk (empty if there is none)"""
    if not os.path.exists(OUT) or not os.path.exists(MANIFEST):
        return ()
    try:
        with open(MANIFEST) as f:
            return tuple(json.load(f)["components"])
    except (OSError, ValueError, KeyError):
        return ()


def _deps():
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [
        os.path.join(HERE, "..", "include", "asd_b200.h"), os.path.abspath(__file__)]


def needs_build(components=None) -> bool:
    want = _closure(components if components is not None else all_components())
    have = built_components()
    if not set(want) <= set(have):
        return True
    t = os.path.getmtime(OUT)
    return any(os.path.getmtime(d) > t for d in _deps())


def build(force: bool = False, verbose: bool = False, components=None) -> str:
    if not force and not needs_build(components):
        return OUT
    # keep what the library already holds: a later, wider request never drops a component
    comps = _closure(tuple(components if components is not None else all_components()) +
                     tuple(c for c in built_components() if c in COMPONENTS))
    objs = []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    procs = []
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if not f.endswith(".cu")] + [
        os.path.join(HERE, "..", "include", "asd_b200.h")]
    newest_header = max(os.path.getmtime(h) for h in headers)
    for src in sources(comps):
        obj = os.path.join(HERE, "build", os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(src), newest_header):
            continue
        cmd = [NVCC, *FLAGS, "-c", src, "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        log = os.path.join(HERE, "build", os.path.basename(src)[:-3] + ".ptxas.log")
        with open(log, "w") as f:
            f.write(out)
    tmp = OUT + f".{os.getpid()}.tmp"
    cmd = [NVCC, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart_static",
           "-ldl", "-lpthread", "-lrt"]
    subprocess.check_call(cmd)
    os.replace(tmp, OUT)
    with open(MANIFEST, "w") as f:
        json.dump({"components": list(comps)}, f)
    return OUT


if __name__ == "__main__":
    only = [a.split("=", 1)[1].split(",") for a in sys.argv if a.startswith("--components=")]
    print(build(force="--force" in sys.argv, verbose=True, components=only[0] if only else None))
