"""Builds the native front end in-tree with g++: ``tgi-b200-router`` (HTTP + scheduler, embeds
CPython for the tokenizer bridge), ``tgi-b200-launcher`` (process supervisor), ``tgi-b200-benchmark`` (shard-level prefill/decode
microbenchmark) and ``_router_test.so``
(pybind11 bindings of the scheduler core that the unit tests drive)."""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "src"
OBJ = HERE / "_build"
CXX = os.environ.get("CXX", "g++")
FLAGS = ["-std=c++17", "-O2", "-g", "-fPIC", "-Wall", "-pthread"]
CORE = ["pb.cpp", "scheduler.cpp", "shard_client.cpp", "trace.cpp", "usage.cpp", "http.cpp", "images.cpp", "api.cpp", "api_routes.cpp", "api_openai.cpp", "api_kserve.cpp", "openapi.cpp"]


def _py_flags():
    inc = sysconfig.get_paths()["include"]
    libdir = sysconfig.get_config_var("LIBDIR")
    ver = sysconfig.get_config_var("LDVERSION") or sysconfig.get_config_var("VERSION")
    return [f"-I{inc}"], [f"-L{libdir}", f"-lpython{ver}", "-ldl", "-lm"]


def _compile(src: Path, extra):
    obj = OBJ / (src.stem + ".o")
    deps = [src] + list(SRC.glob("*.hpp"))
    if obj.exists() and all(d.stat().st_mtime <= obj.stat().st_mtime for d in deps):
        return obj
    cmd = [CXX, *FLAGS, *extra, "-I", str(SRC), "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"{' '.join(cmd)}\n{r.stderr}")
    return obj


def build(tests: bool = True):
    OBJ.mkdir(exist_ok=True)
    py_inc, py_ld = _py_flags()
    import pybind11

    jobs = [(SRC / f, []) for f in CORE] + [(SRC / "pybridge.cpp", py_inc), (SRC / "main.cpp", []),
                                            (SRC / "launcher.cpp", []), (SRC / "benchmark.cpp", [])]
    if tests:
        jobs.append((SRC / "bindings.cpp", py_inc + [f"-I{pybind11.get_include()}"]))
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        objs = dict(zip([j[0].stem for j in jobs], ex.map(lambda j: _compile(*j), jobs)))
    core = [str(objs[Path(f).stem]) for f in CORE]

    def link(out, parts, extra):
        cmd = [CXX, "-o", str(out), *parts, "-pthread", *extra]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"{' '.join(cmd)}\n{r.stderr}")

    link(HERE / "tgi-b200-router", core + [str(objs["pybridge"]), str(objs["main"])], py_ld)
    link(HERE / "tgi-b200-launcher", [str(objs["launcher"])], [])
    link(HERE / "tgi-b200-benchmark", [str(objs[n]) for n in ("pb", "scheduler", "shard_client", "trace", "benchmark")], [])
    if tests:
        link(HERE / "_router_test.so", core + [str(objs["bindings"])], ["-shared"])
    return HERE / "tgi-b200-router"


if __name__ == "__main__":
    print(build())
