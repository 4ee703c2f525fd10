"""Compiles tests/cpp/test_header_layer.cpp against include/anygpu, libanygpu_b200.so and liboracle.so."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "_build", "test_header_layer")


def build():
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    src = os.path.join(HERE, "test_header_layer.cpp")
    libdir, orcdir = os.path.join(ROOT, "anygpu_b200", "lib"), os.path.join(ROOT, "oracle")
    cmd = [os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc"), "-std=c++17", "-O2", "-x", "cu", "-DAC_WITH_ASSERT",
           "-gencode", "arch=compute_100a,code=sm_100a", "-I", os.path.join(ROOT, "include"), src, "-o", OUT,
           "-L", libdir, "-lanygpu_b200", "-L", orcdir, "-loracle",
           "-Xlinker", "-rpath=$ORIGIN/../../../anygpu_b200/lib", "-Xlinker", "-rpath=$ORIGIN/../../../oracle"]
    subprocess.check_call(cmd)
    return OUT


SFT_OUT = os.path.join(HERE, "_build", "sft_dump")


def build_sft_dump():
    """Host-only program around the safetensors reader (compiled with nvcc for the CUDA headers tensor.hpp includes)."""
    os.makedirs(os.path.dirname(SFT_OUT), exist_ok=True)
    cmd = [os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc"), "-std=c++17", "-O1", "-x", "cu", "-DAC_WITH_ASSERT",
           "-gencode", "arch=compute_100a,code=sm_100a", "-I", os.path.join(ROOT, "include"), os.path.join(HERE, "sft_dump.cpp"),
           "-o", SFT_OUT]
    subprocess.check_call(cmd)
    return SFT_OUT


if __name__ == "__main__":
    print(build())
    print(build_sft_dump())
