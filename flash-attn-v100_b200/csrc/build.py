"""Build libfa_b200.so for sm_100a with bare nvcc (no torch headers needed).

Usage: python build.py [--force] [--verbose]
The library lands in ../flash_attention_v100/lib/ so it travels with the package.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(os.path.dirname(HERE), "flash_attention_v100", "lib")
OUT = os.path.join(OUT_DIR, "libfa_b200.so")
SOURCES = ["host_api.cu", "simt_kernels.cu", "fwd_sm100.cu", "fwd_tf32_sm100.cu", "bwd_sm100.cu", "combine.cu"]
HEADERS = ["fa_common.cuh", "philox.cuh", "sm100_ptx.cuh", "tma_host.cuh", "tile_config.cuh",
           os.path.join("..", "..", "include", "fa_b200.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--use_fast_math", "-Xptxas", "-v",
]


def _newest(paths):
    return max((os.path.getmtime(p) for p in paths if os.path.exists(p)), default=0.0)


def build(force=False, verbose=False):
    os.makedirs(OUT_DIR, exist_ok=True)
    srcs = [os.path.join(HERE, s) for s in SOURCES]
    deps = srcs + [os.path.join(HERE, h) for h in HEADERS] + [os.path.abspath(__file__)]
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= _newest(deps):
        return OUT
    nvcc = os.environ.get("NVCC", "nvcc")
    objs = []
    procs = []
    for s in srcs:
        o = os.path.join(OUT_DIR, os.path.basename(s).replace(".cu", ".o"))
        objs.append(o)
        flags = list(NVCC_FLAGS)
        if os.path.basename(s) == "simt_kernels.cu":
            flags.remove("--use_fast_math")  # exact expf/logf/division in the fp32 family
        cmd = [nvcc] + flags + ["-c", s, "-o", o]
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    log = []
    for cmd, pr in procs:
        out, _ = pr.communicate()
        log.append(" ".join(cmd) + "\n" + out)
        if pr.returncode != 0:
            sys.stderr.write("\n".join(log))
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    link = [nvcc, "-shared", "-o", OUT] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    log.append(" ".join(link) + "\n" + r.stdout)
    if r.returncode != 0:
        sys.stderr.write("\n".join(log))
        raise RuntimeError("link failed")
    with open(os.path.join(OUT_DIR, "build.log"), "w") as f:
        f.write("\n".join(log))
    if verbose:
        print("\n".join(log))
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
