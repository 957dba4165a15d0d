"""The C++ adapter against the reference's own interface headers (CPU: compile and link only).

Where the reference tree is mounted, cl-eden-kernel_b200/adapter/b200_operators.cpp and tests/adapter_test.cpp are built
with -DENN_B200_WITH_REFERENCE_HEADERS: Status / Dim4 / DataType ... from Common.hpp, ActivationInfo, the full ITensor
(B200Tensor overrides every pure virtual or the build fails as abstract), Parameters / Pool2DParameters from
CLParameter.hpp and the parameter structs from the CL* operator headers replace the stand-in declarations.  The binary
stays beside the tests; the GPU suite runs it when it is there.
"""
import os
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
PKG = os.path.join(ROOT, "cl-eden-kernel_b200")
REF_SRC = "/root/reference/src"
REF_EXE = os.path.join(HERE, "adapter_test_refhdr.bin")


def ref_flags():
    stub = os.path.join(REF_SRC, "userdriver/gpu/third_party/opencl_stub")
    return ["-DENN_B200_WITH_REFERENCE_HEADERS", "-Wno-subobject-linkage", "-I" + REF_SRC, "-I" + stub, "-I" + os.path.join(stub, "CL")]


def test_adapter_builds_standalone(tmp_path):
    for src in (os.path.join(PKG, "adapter", "b200_operators.cpp"), os.path.join(HERE, "adapter_test.cpp")):
        r = subprocess.run(["/usr/bin/g++", "-std=c++17", "-Wall", "-c", "-o", str(tmp_path / "a.o"), src], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr


@pytest.mark.skipif(not os.path.isdir(REF_SRC), reason="reference tree not mounted")
def test_adapter_builds_against_reference_headers():
    subprocess.run(["make", "-C", PKG], check=True, capture_output=True)
    subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "liboracle.so"], check=True, capture_output=True)
    r = subprocess.run(["/usr/bin/g++", "-O1", "-std=c++17", "-Wall", *ref_flags(), "-o", REF_EXE,
                        os.path.join(HERE, "adapter_test.cpp"), os.path.join(PKG, "adapter", "b200_operators.cpp"),
                        "-L" + PKG, "-lenn_b200", "-L" + os.path.join(ROOT, "oracle"), "-loracle",
                        "-Wl,-rpath,$ORIGIN/../cl-eden-kernel_b200", "-Wl,-rpath,$ORIGIN/../oracle", "-fopenmp"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    # the reference's ITensor really is the base class: a tensor of this driver converts to the reference's pointer type
    probe = r'''
#include "%s/adapter/b200_operators.hpp"
#include <type_traits>
static_assert(std::is_base_of<::enn::ud::ITensor, ::enn::ud::b200::B200Tensor>::value, "B200Tensor is an enn::ud::ITensor");
static_assert(!std::is_abstract<::enn::ud::b200::B200Tensor>::value, "every ITensor member is implemented");
static_assert(std::is_same<::enn::ud::b200::ConvolutionParameters, ::enn::ud::gpu::ConvolutionParameters>::value, "reference parameter struct");
static_assert(std::is_same<::enn::ud::b200::Pool2DParameters, ::enn::ud::gpu::Pool2DParameters>::value, "reference parameter struct");
static_assert(std::is_same<::enn::ud::b200::Status, ::Status>::value, "reference Status");
int main() { return 0; }
''' % PKG
    r = subprocess.run(["/usr/bin/g++", "-std=c++17", "-fsyntax-only", *ref_flags(), "-x", "c++", "-"], input=probe, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
