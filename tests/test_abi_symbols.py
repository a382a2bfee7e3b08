"""The C ABI library loads and exports every symbol the headers declare, and every THNN_Cuda* /
THNN_CudaDouble* name the reference's FFI binding looks up.  No GPU needed: nothing is computed."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared(header):
    src = open(os.path.join(ROOT, "include", header)).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"CUNN_API\s+[A-Za-z_0-9 \*]+?\b([A-Za-z_0-9]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    from cunn_b200._lib import lib, SO_PATH
    assert os.path.exists(SO_PATH)
    names = declared("cunn_b200.h") + declared("THCUNN_b200.h") + declared("cunn_b200_dpt.h")
    assert len(names) > 60
    for n in names:
        assert hasattr(lib, n), n


def test_library_exports_all_reference_binding_names():
    # the names THCUNN.lua extracts from generic/THCUNN.h (regenerate with cunn_b200/csrc/gen_thnn_names.py)
    from cunn_b200._lib import lib
    inc = open(os.path.join(ROOT, "cunn_b200", "csrc", "thnn_names.inc")).read()
    names = re.findall(r"^X\(([A-Za-z0-9_]+)\)", inc, flags=re.M)
    assert len(names) == 162
    for n in names:
        for typ in ("Cuda", "CudaDouble"):
            assert hasattr(lib, "THNN_" + typ + n), n


def test_unimplemented_entry_point_reports_through_the_error_hook():
    from cunn_b200 import thnn
    nnb = thnn.THNN()
    f = thnn.lib.THNN_CudaAbs_updateOutput
    f.restype = None
    f.argtypes = [ctypes.c_void_p]
    f(nnb.state)
    assert nnb.errors and "THNN_CudaAbs_updateOutput is not implemented" in nnb.errors[-1]
    nnb.close()


def test_no_cpu_fallback_message():
    # without a device the compute entry points fail with a CUDA error instead of computing anything
    import torch
    if torch.cuda.is_available():
        return
    from cunn_b200._lib import lib
    rc = lib.cunn_b200_threshold_forward(ctypes.c_void_p(16), ctypes.c_void_p(16), 4, 0.0, 0.0, None)
    assert rc != 0 and lib.cunn_b200_last_error()


def test_cutorch_backend_of_the_entry_points_compiles(tmp_path):
    """csrc/thnn.cu built with -DCUNN_B200_USE_REAL_THC against a header that only DECLARES cutorch's
    functions (tests/thc_stub): the object must leave exactly the libTHC calls the reference's wrappers use
    as undefined symbols, and still define every THNN_Cuda* entry point of the hot path."""
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        import pytest
        pytest.skip("nvcc not available")
    obj = str(tmp_path / "thnn_real.o")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O0", "-std=c++17", "-ccbin", "/usr/bin/g++",
           "-Xcompiler", "-fPIC", "-DCUNN_BUILDING=1", "-DCUNN_B200_USE_REAL_THC",
           "-I", os.path.join(ROOT, "tests", "thc_stub"), "-c", os.path.join(ROOT, "cunn_b200", "csrc", "thnn.cu"), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    syms = subprocess.run(["nm", obj], capture_output=True, text=True, check=True).stdout.splitlines()
    undefined = {l.split()[-1] for l in syms if " U " in l}
    defined = {l.split()[-1] for l in syms if " T " in l}
    thc = {n for n in undefined if n.startswith(("THC", "_THError"))}
    assert thc == {"THCState_getCurrentStream", "THCudaMalloc", "THCudaFree", "THCudaTensor_new", "THCudaTensor_free",
                   "THCudaTensor_newContiguous", "THCudaTensor_resizeNd", "THCudaLongTensor_resizeNd", "_THError",
                   "THCudaDoubleTensor_free", "THCudaDoubleTensor_newContiguous", "THCudaDoubleTensor_resizeNd"} - \
        ({"THCudaTensor_new"} - thc)
    for n in ("THNN_CudaSpatialDepthWiseConvolution_updateOutput", "THNN_CudaSpatialConvolutionMM_accGradParameters",
              "THNN_CudaBatchNormalization_backward", "THNN_CudaSpatialMaxPooling_updateOutput",
              "THNN_CudaDoubleSpatialDepthWiseConvolution_updateOutput", "THNN_CudaDoubleBatchNormalization_backward"):
        assert n in defined
    assert not any(n.startswith("THCState_b200") for n in defined)      # the harness layer is built-in only
