#!/usr/bin/env python3
"""Build the upstream project's dense Qwen3 path, unmodified, for sm_100a, with a small driver.

Upstream ships one CMake target (`runner`, CMakeLists.txt:12-35) built for sm_120a whose `main()`
(inference.cpp:54-65) instantiates the mixture-of-experts classes only.  The dense classes take
everything they need as arguments (`Qwen3::from_pretrained`, src/models/qwen3/qwen3.cpp:42-112;
`KVCache`, src/kvcache.h:40-61; `FlashAttnEngine`, src/src-cuda/attention/fattn.cuh:33-46), so this
script compiles upstream's own source files as they are (read from the upstream checkout, never
copied or edited) with upstream's flags except the architecture, and links them with
`reference_driver.cpp`, which does what upstream's `main()` does around the dense classes.

Left out of the link because the dense path never reaches them: the tokenizer, the mixture-of-experts
model, its CPU expert runtime and `model.cpp` (the registry, which pulls those in).

    python baseline/build_reference.py [--src UPSTREAM_DIR] [--out baseline/_ref] [--jobs N]

The result is `<out>/bin/reference_runner`.  Object files are kept, so a second call only links.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import os
import subprocess
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent

# upstream's translation units on the dense path (CMakeLists.txt:8-18 globs every file; these are the
# ones the dense classes and the driver reference)
SOURCES = [
    "src/models/qwen3/qwen3.cpp",
    "src/src-cuda/tensor.cu",
    "src/src-cuda/embedding.cu",
    "src/src-cuda/norm.cu",
    "src/src-cuda/rope.cu",
    "src/src-cuda/kvcache.cu",
    "src/src-cuda/attention/fattn.cu",
    "src/src-cuda/mat-ops/mat-ops.cu",
    "src/src-cuda/mat-ops/gemm/gemm.cu",
    "src/src-cuda/mat-ops/gemm/gemm-fp8.cu",
    "src/src-cuda/mat-ops/simple-ops/hadamard.cu",
    "src/src-cuda/mat-ops/simple-ops/matrix-add.cu",
    "src/src-cuda/quantization/quant.cu",
    "src/src-cuda/activations/silu.cu",
    "src/src-cuda/simple-ops/simple-ops.cu",
    "src/src-cuda/reductions/argmax.cu",
]

# CMakeLists.txt:47-63: every directory that holds a header, plus the vendored trees
INCLUDES = [
    "src", "src/src-cuda", "src/tokenizers", "src/models", "src/models/qwen3", "src/models/qwen3_moe",
    "src/src-cuda/activations", "src/src-cuda/attention", "src/src-cuda/mat-ops", "src/src-cuda/moe",
    "src/src-cuda/quantization", "src/src-cuda/reductions", "src/src-cuda/simple-ops",
    "src/moe-managers", "src/src-cpu", "src/external", "src/external/cudnn-frontend/include",
]


def nvcc_flags(src: Path) -> list[str]:
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-w", "-rdc=true",
             "-Xcompiler", "-pthread", "-x", "cu"]
    for inc in INCLUDES:
        flags += ["-I", str(src / inc)]
    return flags


def compile_one(nvcc: str, src: Path, rel: str, obj: Path) -> tuple[str, float, int, str]:
    t0 = time.time()
    obj.parent.mkdir(parents=True, exist_ok=True)
    cmd = [nvcc, *nvcc_flags(src), "-c", str(src / rel), "-o", str(obj)]
    p = subprocess.run(cmd, capture_output=True, text=True)
    return rel, time.time() - t0, p.returncode, p.stderr[-4000:]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", default=os.environ.get("GARLIC_REFERENCE_SRC", str(HERE.parent.parent / "reference")),
                    help="upstream's checkout (default: $GARLIC_REFERENCE_SRC, else a folder `reference` beside this repository)")
    ap.add_argument("--out", default=str(HERE / "_ref"))
    ap.add_argument("--jobs", type=int, default=max(1, (os.cpu_count() or 2) - 1))
    ap.add_argument("--force", action="store_true", help="recompile objects that exist")
    args = ap.parse_args()
    src, out = Path(args.src), Path(args.out)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    if not (src / "src/models/qwen3/qwen3.cpp").is_file():
        print(f"build_reference: no upstream checkout at {src}", file=sys.stderr)
        return 3
    (out / "obj").mkdir(parents=True, exist_ok=True)
    (out / "bin").mkdir(parents=True, exist_ok=True)

    jobs = []
    for rel in SOURCES:
        obj = out / "obj" / (rel.replace("/", "__") + ".o")
        newest = (src / rel).stat().st_mtime
        if args.force or not obj.is_file() or obj.stat().st_mtime < newest:
            jobs.append((rel, obj))
    driver_src = HERE / "reference_driver.cpp"
    driver_obj = out / "obj" / "reference_driver.o"
    print(f"build_reference: {len(jobs)} of {len(SOURCES)} upstream files to compile "
          f"(the attention file alone takes a few minutes)", flush=True)
    with concurrent.futures.ThreadPoolExecutor(args.jobs) as pool:
        futs = [pool.submit(compile_one, nvcc, src, rel, obj) for rel, obj in jobs]
        for f in concurrent.futures.as_completed(futs):
            rel, dt, rc, err = f.result()
            print(f"  {rel}: {dt:.0f} s, rc {rc}", flush=True)
            if rc:
                print(err, file=sys.stderr)
                return 1
    p = subprocess.run([nvcc, *nvcc_flags(src), "-I", str(HERE), "-c", str(driver_src), "-o", str(driver_obj)],
                       capture_output=True, text=True)
    if p.returncode:
        print(p.stderr[-6000:], file=sys.stderr)
        return 1
    objs = [str(out / "obj" / (rel.replace("/", "__") + ".o")) for rel in SOURCES] + [str(driver_obj)]
    exe = out / "bin" / "reference_runner"
    # CMakeLists.txt:35: cublas cublasLt cudnn nvrtc pthread nvidia-ml
    link = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-rdc=true", *objs, "-o", str(exe),
            "-lcublas", "-lcublasLt", "-lcudnn", "-lnvrtc", "-lpthread", "-L/usr/local/cuda/lib64/stubs", "-lnvidia-ml"]
    p = subprocess.run(link, capture_output=True, text=True)
    if p.returncode:
        print(p.stderr[-6000:], file=sys.stderr)
        return 1
    print(f"build_reference: {exe}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
