"""Builds libyaxus_cuda.so (sm_100a) and the host-side library in-tree with nvcc / g++."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libyaxus_cuda.so")
HOST_OUT = os.path.join(HERE, "libyaxus_host.so")
TRACE_OUT = os.path.join(HERE, "libyaxus_cuda_trace.so")
CUDA_SOURCES = ["api.cu", "kv_ops.cu", "attend_simt.cu", "attend_mma.cu", "prefill_tc.cu", "combine.cu", "dist.cu", "attend_static.cu", "model_ops.cu", "planner.cpp",
                "hooks.cu"]
HOST_SOURCES = [os.path.join("host", "kv_cache.cpp")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-Wall,-Wno-unknown-pragmas", "--expt-relaxed-constexpr",
]


def _stale(out, deps):
    return not os.path.exists(out) or any(os.path.getmtime(d) > os.path.getmtime(out) for d in deps)


def _deps(sources):
    deps = [os.path.join(CSRC, s) for s in sources]
    for root, _, files in os.walk(CSRC):
        deps += [os.path.join(root, f) for f in files if f.endswith((".h", ".hpp", ".cuh"))]
    deps.append(os.path.join(HERE, "..", "include", "yaxus_cuda.h"))
    return deps


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    """Compiles every CUDA source for sm_100a into yaxus_b200/libyaxus_cuda.so.  With `trace`
    the kernels' diagnostic time stamps are compiled in (-DYX_TRACE) and the result goes to
    libyaxus_cuda_trace.so instead; YAXUS_CUDA_LIB=<that path> makes the bindings load it."""
    target = TRACE_OUT if trace else OUT
    if force or _stale(target, _deps(CUDA_SOURCES)):
        objs = []
        os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
        procs = []
        for s in CUDA_SOURCES:
            obj = os.path.join(HERE, "build", s.replace("/", "_") + (".trace.o" if trace else ".o"))
            objs.append(obj)
            cmd = ["nvcc", *NVCC_FLAGS, *(["-DYX_TRACE"] if trace else []), "-x", "cu", "-c", os.path.join(CSRC, s), "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        failed = False
        for s, p in procs:
            out, _ = p.communicate()
            if p.returncode != 0 or verbose:
                print(f"--- {s}\n{out}")
            failed |= p.returncode != 0
        if failed:
            raise RuntimeError("nvcc failed")
        subprocess.run(["nvcc", "-shared", "-o", target, *objs, "-ldl"], check=True)
    if trace:
        return target
    if force or _stale(HOST_OUT, _deps(HOST_SOURCES)):
        cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-Wall", "-o", HOST_OUT,
               *[os.path.join(CSRC, s) for s in HOST_SOURCES]]
        subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv))
