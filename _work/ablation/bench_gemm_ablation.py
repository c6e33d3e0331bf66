"""Where the time of the block-fp8 GEMM goes: the same kernel with parts switched off.

``gemm_sm100.cu`` compiles, under ``-DTGI_GEMM_EXP``, three switches into the kernel (they change the
result, so they exist only in this separately built library, ``_build/libgemm_exp.so``):

====  ==========================================================================================
mode  what still runs
====  ==========================================================================================
0     everything (the production kernel)
1     no promotion FMAs (TMEM loads, MMAs, TMA pipeline stay)
2     no TMEM loads either (MMAs and the TMA pipeline stay)
3     no MMAs either: only the TMA pipeline and its barriers, i.e. the operand traffic into shared memory
====  ==========================================================================================

Usage (one GPU)::

    python -m tgi_b200.ops.bench_gemm_ablation                       # decode and prefill shapes of Llama-3-70B
    python -m tgi_b200.ops.bench_gemm_ablation --shape 256,57344,8192 --modes 0,3

Timing: CUDA events around direct launches (median of ``--iters``), after warm-up; the operands are larger
than L2 for the default shapes.  One JSON line per (shape, mode).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import subprocess
from pathlib import Path

import torch

from .build import BUILD_DIR, CSRC, NVCC_FLAGS, nvcc_path


def build_exp_library() -> Path:
    BUILD_DIR.mkdir(exist_ok=True)
    out = BUILD_DIR / "libgemm_exp.so"
    src = CSRC / "gemm_sm100.cu"
    deps = [src] + sorted(CSRC.glob("*.cuh"))
    if out.exists() and all(d.stat().st_mtime <= out.stat().st_mtime for d in deps):
        return out
    cmd = [nvcc_path(), *NVCC_FLAGS, "-DTGI_GEMM_EXP", "-I", str(CSRC), "-shared", str(src), "-o", str(out),
           "-lcudart_static", "-ldl", "-lrt", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{r.stderr}")
    return out


def run_shape(lib, M: int, N: int, K: int, modes, iters: int, dev) -> None:
    xq = torch.randint(0, 100, (M, K), device=dev, dtype=torch.uint8)
    wq = torch.randint(0, 100, (N, K), device=dev, dtype=torch.uint8)
    pitch = (M + 3) & ~3
    xs = torch.rand(K // 128, pitch, device=dev) * 0.01
    wsc = torch.rand((N + 127) // 128, K // 128, device=dev) * 0.01
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    ctas = torch.cuda.get_device_properties(dev).multi_processor_count
    ws = torch.empty(lib.tgi_gemm_workspace_floats(M, ctas), device=dev, dtype=torch.float32)
    cnt = torch.zeros(65536, device=dev, dtype=torch.int32)
    st = torch.zeros(1, device=dev, dtype=torch.int32)
    stream = torch.cuda.current_stream().cuda_stream
    p = lambda t: ctypes.c_void_p(t.data_ptr())

    def call():
        rc = lib.tgi_gemm_fp8_block(p(xq), p(xs), pitch, p(wq), p(wsc), p(out), None, M, N, K, ctas, p(ws), p(cnt), p(st),
                                    ctypes.c_void_p(stream))
        if rc != 0:
            raise RuntimeError(f"tgi_gemm_fp8_block returned {rc}")

    for mode in modes:
        lib.tgi_gemm_set_exp(mode)
        torch.cuda.synchronize()
        for _ in range(3):
            call()
        times = []
        for _ in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            call()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3)
        times.sort()
        print(json.dumps({"M": M, "N": N, "K": K, "mode": mode, "median_us": round(times[len(times) // 2], 1),
                          "min_us": round(times[0], 1), "kernel_status": int(st.item()),
                          "weight_bytes": N * K, "hbm_floor_us_at_6.65TBs": round(N * K / 6.65e6, 1)}), flush=True)
        st.zero_()
        cnt.zero_()
    lib.tgi_gemm_set_exp(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", action="append", help="M,N,K (repeatable)")
    ap.add_argument("--modes", default="0,1,2,3")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    shapes = [tuple(int(v) for v in s.split(",")) for s in (args.shape or [])] or [
        (256, 57344, 8192), (256, 8192, 28672), (4096, 8192, 8192)]
    lib = ctypes.CDLL(str(build_exp_library()))
    lib.tgi_gemm_workspace_floats.restype = ctypes.c_longlong
    dev = torch.device("cuda", 0)
    for M, N, K in shapes:
        run_shape(lib, M, N, K, [int(m) for m in args.modes.split(",")], args.iters, dev)


if __name__ == "__main__":
    main()
