"""Build libanalog_b200.so (sm_100a) in-tree with nvcc.

    python aihwkit-lightning_b200/build.py [--force]

The library lands in ``aihwkit_lightning_b200/lib/`` next to the Python package that loads it
with ctypes.  nvcc cross-compiles without a GPU.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "aihwkit_lightning_b200", "lib")
OUT = os.path.join(OUT_DIR, "libanalog_b200.so")
SOURCES = [
    "api.cu",
    "reduce_kernels.cu",
    "prepass_kernels.cu",
    "split_kernels.cu",
    "gemm_simt.cu",
    "gemm_tcgen05_fwd.cu",
    "gemm_tcgen05_bwd.cu",
    "gemm_smallm.cu",
    "backward_kernels.cu",
    "conv_kernels.cu",
    "peer_kernels.cu",
    "decoder_glue_kernels.cu",
]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17", "--expt-relaxed-constexpr", "--extended-lambda",
    "-Xcompiler", "-fPIC,-ffp-contract=off",
    "-Xptxas", "-v",
]


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    built = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(HERE, "..", "include", "analog_b200.h"))
    return any(os.path.getmtime(p) > built for p in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(OUT_DIR, src.replace(".cu", ".o"))
        objs.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    log = []
    for src, proc in procs:
        out, _ = proc.communicate()
        log.append(f"==== {src}\n{out}")
        if proc.returncode != 0:
            sys.stderr.write("\n".join(log))
            raise RuntimeError(f"nvcc failed on {src}")
    with open(os.path.join(OUT_DIR, "ptxas.log"), "w") as fh:
        fh.write("\n".join(log))
    link = [nvcc, "-shared", "-o", OUT, *objs, "-lcudart", "-ldl"]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("link failed")
    if verbose:
        print("\n".join(log))
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
