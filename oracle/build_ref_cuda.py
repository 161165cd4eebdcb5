"""Compiles the reference's own CUDA library for sm_100a (checker / baseline only).

    python oracle/build_ref_cuda.py [--ref /path/to/arboretum] [--tests]

TEST INFRASTRUCTURE ONLY.  The sources are read where they lie in the reference
tree, copied to a scratch directory outside this repository, given the five small
compatibility edits the reference needs to compile with CUDA 12.9 (none of them
changes arithmetic), and compiled with nvcc.  Only binaries are written here:

    oracle/_ref/libarboretum_ref.so   the 14 entry points of python-wrapper/arboretum_wrapper.h
    oracle/_ref/ref_kats              (--tests) the reference's tests/cpp known-answer tests for
                                      the quantizer, the partition index and the histogram sums,
                                      built against a minimal stand-in for googletest

The compatibility edits:
  1. src/core/cuda_helpers.h:145-148: `void atomicAdd(float2 *, float2)` collides with the
     toolkit's own `float2 atomicAdd(float2 *, float2)` (same component-wise float adds); the
     reference's overload is renamed out of the way and the calls bind to the toolkit's.
  2. thrust/system/cuda/experimental/pinned_allocator.h no longer exists: a header of that
     name in oracle/ref_cuda_compat/ provides the allocator over cudaMallocHost.
  3. `using namespace thrust;` makes `cub::` ambiguous with `thrust::cub`: every `cub::`
     becomes `::cub::`, and the directive becomes using-declarations of the names used.
  4. Device-side cudaDeviceSynchronize() was removed from CUDA 12: the calls in
     hist_tree_grower.cu:78, continuous_tree_grower.cu:90 and builder.h:161,167 are dropped
     (child grids still finish before their parent grid does; nothing in the parent reads
     their output).
  5. cub::DeviceReduce::Sum over float2 into mydouble2 needs `operator+` for the mixed
     pairs that CUB's accumulator deduction forms: added beside the existing operators.
"""
import argparse
import glob
import os
import re
import shutil
import subprocess
import sys
import tempfile
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
COMPAT = os.path.join(HERE, "ref_cuda_compat")
NVCC = os.environ.get("NVCC", "nvcc")
FLAGS = ["-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-rdc=true", "-O3", "-w",
         "--expt-extended-lambda", "--default-stream", "per-thread", "-Xcompiler", "-fPIC,-fopenmp,-O3",
         "-ccbin", "/usr/bin/g++"]


# the names the reference takes from namespace thrust, imported one by one: a global
# `using namespace thrust;` also drags in thrust::cub, and the kernel stubs nvcc generates
# for the translation unit then find `cub::` ambiguous
USING_THRUST = ("using thrust::host_vector; using thrust::device_vector; using thrust::raw_pointer_cast; "
                "using thrust::device_ptr; using thrust::device_pointer_cast; using thrust::counting_iterator;")


def find_json_header():
    import sysconfig
    for base in (sysconfig.get_paths()["purelib"], "/usr/include", "/usr/local/include"):
        for p in glob.glob(os.path.join(base, "**", "nlohmann", "json.hpp"), recursive=True):
            return os.path.dirname(p)
    raise SystemExit("nlohmann/json.hpp not found (the reference's _json submodule is empty)")


def patch(text, name):
    text = re.sub(r"(?<![:\w])cub::", "::cub::", text)                         # edit 3
    text = text.replace("using namespace thrust;", USING_THRUST)
    if name in ("hist_tree_grower.cu", "continuous_tree_grower.cu", "builder.h"):  # edit 4
        text = text.replace("DEVICE_OK(cudaDeviceSynchronize());", "")
    if name == "cuda_helpers.h":
        text = text.replace("__forceinline__ __device__ void atomicAdd(float2 *address",
                            "__forceinline__ __device__ void atomicAdd_unused(float2 *address")  # edit 1
        text = text.replace("#endif  // SRC_CORE_CUDA_HELPERS_H",                           # edit 5
                            '#include "ref_mixed_sums.h"\n#endif  // SRC_CORE_CUDA_HELPERS_H')
    return text


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("REF", ""), help="the reference tree (or REF=...)")
    ap.add_argument("--tests", action="store_true")
    ap.add_argument("--keep", action="store_true", help="keep the scratch directory")
    args = ap.parse_args()
    if not os.path.isdir(os.path.join(args.ref, "src", "core")):
        raise SystemExit("reference tree not found at %s" % args.ref)
    os.makedirs(OUT, exist_ok=True)
    work = tempfile.mkdtemp(prefix="arboretum_ref_build_")
    try:
        for sub in ("src/core", "src/io", "python-wrapper", "tests/cpp"):
            os.makedirs(os.path.join(work, sub))
            for p in sorted(glob.glob(os.path.join(args.ref, sub, "*"))):
                with open(p) as f:
                    text = f.read()
                with open(os.path.join(work, sub, os.path.basename(p)), "w") as f:
                    f.write(patch(text, os.path.basename(p)))
        inc = ["-I" + os.path.join(work, "src"), "-I" + os.path.join(work, "src", "core"), "-I" + COMPAT,
               "-I" + find_json_header()]
        sources = sorted(glob.glob(os.path.join(work, "src", "core", "*.cu")) +
                         glob.glob(os.path.join(work, "src", "core", "*.cpp")) +
                         glob.glob(os.path.join(work, "src", "io", "*.cu")) +
                         glob.glob(os.path.join(work, "python-wrapper", "*.cu")))
        tests = []
        if args.tests:
            tests = [os.path.join(work, "tests", "cpp", t) for t in
                     ("test_datamatrix.cu", "test_hist_sum.cu", "test_hist.cu", "test_helpers.cu")]
            tests.append(os.path.join(COMPAT, "kat_main.cu"))

        def compile_one(src):
            obj = os.path.join(work, os.path.basename(src) + ".o")
            cmd = [NVCC] + FLAGS + inc + (["-x", "cu"] if src.endswith(".cpp") else []) + ["-c", src, "-o", obj]
            r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed for %s:\n%s" % (src, r.stdout[-6000:]))
            return obj

        with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
            objs = list(ex.map(compile_one, sources))
            test_objs = list(ex.map(compile_one, tests))
        lib = os.path.join(OUT, "libarboretum_ref.so")
        link = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", lib] + objs + \
               ["-lcudadevrt", "-lgomp", "-ccbin", "/usr/bin/g++"]
        subprocess.check_call(link)
        print(lib)
        if args.tests:
            exe = os.path.join(OUT, "ref_kats")
            wrapper = os.path.join(work, "arboretum_wrapper.cu.o")
            link = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-o", exe] + \
                   [o for o in objs if o != wrapper] + test_objs + ["-lcudadevrt", "-lgomp", "-ccbin", "/usr/bin/g++"]
            subprocess.check_call(link)
            print(exe)
    finally:
        if args.keep:
            print("scratch directory kept:", work)
        else:
            shutil.rmtree(work, ignore_errors=True)


if __name__ == "__main__":
    sys.exit(main())
