"""Builds yinqiwen/lmsf's own CUDA kernels, unmodified, for sm_100a into `baseline/_ref/`.

The reference is a Rust workspace that cannot be built without cargo and a network, but the CUDA
files of its Llama path have torch-free `extern "C"` launchers and compile as they are:

    vllm/kernels/layernorm_kernels.cu       vllm_rms_norm, vllm_fused_add_rms_norm     (:110-187)
    vllm/kernels/pos_encoding_kernels.cu    rotary_embedding                           (:81-167)
    vllm/kernels/cache_kernels.cu           reshape_and_cache                          (:235-290)
    vllm/kernels/activation_kernels.cu      vllm_silu_and_mul                          (:55-127)
    vllm/kernels/attention/attention_kernels.cu   paged_attention_v1 / _v2             (:659-828, :922-1099)

The flags are the reference's own (vllm/build.rs:118-135: -O3, --default-stream per-thread,
--use_fast_math, the -U__CUDA_NO_* switches) with the architecture set to sm_100a.  Nothing is
copied into this repository: the sources are read where the reference lies (`$LMSF_REFERENCE_DIR`, by default the
folder `reference` beside this repository's folder) and only the built library is kept, in a folder that git ignores.

    python baseline/build_ref.py        # builds if needed, prints the library's path
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
SOURCES = ["layernorm_kernels.cu", "pos_encoding_kernels.cu", "cache_kernels.cu", "activation_kernels.cu",
           os.path.join("attention", "attention_kernels.cu")]
FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "--compiler-options", "-fPIC",
         "--default-stream", "per-thread", "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
         "-U__CUDA_NO_HALF2_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "--expt-relaxed-constexpr",
         "--expt-extended-lambda", "--use_fast_math", "-lineinfo"]
LIB_NAME = "libvllm_ref_kernels.so"


class ReferenceUnavailable(RuntimeError):
    pass


def reference_dir() -> str:
    beside = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return os.environ.get("LMSF_REFERENCE_DIR", beside)


def library_path() -> str:
    return os.path.join(OUT_DIR, LIB_NAME)


def _source_hash(kdir: str) -> str:
    h = hashlib.sha256(" ".join(FLAGS).encode())
    for root, _, files in sorted(os.walk(kdir)):
        for f in sorted(files):
            if f.endswith((".cu", ".cuh", ".h")) and "quantization" not in root:
                with open(os.path.join(root, f), "rb") as fh:
                    h.update(f.encode())
                    h.update(fh.read())
    return h.hexdigest()[:16]


def ensure_built(verbose: bool = True) -> str:
    """The path of the built library.  Built here if the reference's sources can be read and the library
    is missing or stale; a library that is already there is used as it is when the sources are not at hand
    (a machine that got the built folder only)."""
    lib, stamp = library_path(), os.path.join(OUT_DIR, "SOURCE_HASH")
    kdir = os.path.join(reference_dir(), "vllm", "kernels")
    have_src = all(os.path.isfile(os.path.join(kdir, s)) for s in SOURCES)
    if not have_src:
        if os.path.isfile(lib):
            return lib
        raise ReferenceUnavailable(f"the reference's kernels are neither built ({lib}) nor readable ({kdir})")
    want = _source_hash(kdir)
    if os.path.isfile(lib) and os.path.isfile(stamp) and open(stamp).read().strip() == want:
        return lib
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isfile(nvcc):
        raise ReferenceUnavailable("nvcc was not found; the reference's kernels cannot be built")
    os.makedirs(OUT_DIR, exist_ok=True)
    objs = []
    for s in SOURCES:
        obj = os.path.join(OUT_DIR, os.path.basename(s)[:-3] + ".o")
        cmd = [nvcc, *FLAGS, "-c", os.path.join(kdir, s), "-o", obj]
        if verbose:
            print(f"[baseline] compiling the reference's {s} for sm_100a ...", file=sys.stderr, flush=True)
        t0 = time.time()
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0:
            raise ReferenceUnavailable(f"nvcc failed on the reference's {s}:\n{p.stdout[-4000:]}")
        if verbose:
            print(f"[baseline]   {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
        objs.append(obj)
    p = subprocess.run([nvcc, "-shared", "-o", lib + ".tmp", *objs, "-lcudart"], stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise ReferenceUnavailable(f"linking the reference's kernels failed:\n{p.stdout[-4000:]}")
    os.replace(lib + ".tmp", lib)
    for o in objs:
        os.remove(o)
    with open(stamp, "w") as f:
        f.write(want + "\n")
    return lib


if __name__ == "__main__":
    print(ensure_built())
