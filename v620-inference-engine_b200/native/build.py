"""Compile the native host library and the C API shim in-tree with g++."""
import glob
import os
import subprocess
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "src")
HOST_LIB = os.path.join(HERE, "libqw_host.so")
ENGINE_LIB = os.path.join(HERE, "libqw_engine.so")
REF_EXE = os.path.join(HERE, "qw_ref")


def _stale(target, deps):
    return not os.path.exists(target) or any(os.path.getmtime(d) > os.path.getmtime(target) for d in deps)


def build(force: bool = False, verbose: bool = False) -> None:
    deps = glob.glob(os.path.join(SRC, "*.hpp")) + glob.glob(os.path.join(SRC, "*.cpp")) + glob.glob(os.path.join(SRC, "*.h"))
    if force or _stale(HOST_LIB, deps):
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-pthread", "-o", HOST_LIB,
               os.path.join(SRC, "host_api.cpp")]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode:
            raise RuntimeError("host library build failed:\n" + r.stdout)
        print("built", HOST_LIB)
    ref_src = os.path.join(HERE, "tools", "qw_ref.cpp")
    if os.path.exists(ref_src) and (force or _stale(REF_EXE, deps + [ref_src])):
        r = subprocess.run(["g++", "-O2", "-std=c++17", "-pthread", "-o", REF_EXE, ref_src], stdout=subprocess.PIPE,
                           stderr=subprocess.STDOUT, text=True)
        if r.returncode:
            raise RuntimeError("qw_ref build failed:\n" + r.stdout)
        print("built", REF_EXE)
    capi = os.path.join(SRC, "capi.cpp")
    if os.path.exists(capi) and (force or _stale(ENGINE_LIB, deps)):
        inc = sysconfig.get_paths()["include"]
        root = os.path.abspath(os.path.join(HERE, "..", ".."))
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-I", inc, "-I", os.path.join(root, "include"),
               "-o", ENGINE_LIB, capi]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode:
            raise RuntimeError("C API shim build failed:\n" + r.stdout)
        print("built", ENGINE_LIB)
