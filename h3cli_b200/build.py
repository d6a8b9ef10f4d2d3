"""Compiles libh3q8.so in-tree for sm_100a with nvcc (cross-compiles without a GPU)."""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libh3q8.so")
PREPARE = os.path.join(HERE, "h3q8_prepare")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-pthread"] + os.environ.get("H3Q8_NVCC_EXTRA", "").split()


def _nvcc():
    for candidate in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    raise RuntimeError("nvcc not found: libh3q8 cannot be built")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    stamp = os.path.getmtime(target)
    return any(os.path.getmtime(s) > stamp for s in sources)


def build(force=False, verbose=False):
    """Builds h3cli_b200/libh3q8.so if any source is newer; returns its path."""
    include = os.path.join(ROOT, "include")
    sources = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC))] + [os.path.join(include, "h3q8.h"), __file__]
    build_dir = os.path.join(HERE, "_build")
    stamp = os.path.join(build_dir, "nvcc_flags.txt")      # a library built with other flags (H3Q8_NVCC_EXTRA) is stale too
    flags = " ".join(NVCC_FLAGS)
    same_flags = os.path.exists(stamp) and open(stamp).read() == flags
    if not force and same_flags and not _stale(LIB, sources):
        return LIB
    os.makedirs(build_dir, exist_ok=True)
    pack_o = os.path.join(build_dir, "q8_pack.o")
    run = lambda cmd: subprocess.run(cmd, check=True, stdout=None if verbose else subprocess.DEVNULL)
    run(["gcc", "-O2", "-std=c11", "-fPIC", "-ffp-contract=off", "-I", include, "-c",
         os.path.join(CSRC, "q8_pack.c"), "-o", pack_o])
    cache_o = os.path.join(build_dir, "q8_cache.o")
    run(["gcc", "-O2", "-std=c11", "-fPIC", "-I", include, "-c", os.path.join(CSRC, "q8_cache.c"), "-o", cache_o])
    plan_o = os.path.join(build_dir, "weight_plan.o")
    run(["gcc", "-O2", "-std=c11", "-fPIC", "-D_GNU_SOURCE", "-I", include, "-c", os.path.join(CSRC, "weight_plan.c"), "-o", plan_o])
    dit_o = os.path.join(build_dir, "dit_linear.o")
    run(["gcc", "-O2", "-std=c11", "-fPIC", "-D_GNU_SOURCE", "-Wall", "-I", include, "-c", os.path.join(CSRC, "dit_linear.c"), "-o", dit_o])
    objects = [pack_o, cache_o, plan_o, dit_o]
    for unit in ("h3q8_raw.cu", "h3_gpu.cu", "h3q8_static.cu", "h3q8_pair_grouped.cu", "h3q8_skinny.cu"):
        obj = os.path.join(build_dir, unit.replace(".cu", ".o"))
        run([_nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-I", include, "-I", CSRC, "-c",
             os.path.join(CSRC, unit), "-o", obj])
        objects.append(obj)
    run([_nvcc(), "-shared", "-o", LIB, *objects, "-lm"])
    with open(stamp, "w") as f:
        f.write(flags)
    # the artifact preparation tool links the library it sits beside
    run(["gcc", "-O2", "-std=c11", "-I", include, os.path.join(CSRC, "q8_prepare.c"), "-o", PREPARE, "-L", HERE, "-lh3q8",
         "-Wl,-rpath,$ORIGIN"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
