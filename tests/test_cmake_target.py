"""The CMake side of the drop-in boundary: a consumer that does what the reference's CMakeLists.txt:88-92, :326-333 does
(add_subdirectory of the tiny-cuda-nn fork, link the target `tiny-cuda-nn`, add ${TCNN_DEFINITIONS}) configures against this
repository.  Configure only: building is covered by the nvcc-based tests."""
import os
import shutil
import subprocess
import sys
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from neus2_b200 import build as B  # noqa: E402

CONSUMER = """cmake_minimum_required(VERSION 3.18)
project(consumer LANGUAGES CXX CUDA)
add_subdirectory("%s" ${CMAKE_BINARY_DIR}/neus2_tcnn)
add_executable(consumer "%s")
target_link_libraries(consumer PUBLIC tiny-cuda-nn)
target_compile_definitions(consumer PUBLIC ${TCNN_DEFINITIONS})
get_target_property(INC tiny-cuda-nn INTERFACE_INCLUDE_DIRECTORIES)
message(STATUS "TCNN_DEFINITIONS=${TCNN_DEFINITIONS}")
message(STATUS "TCNN_INCLUDES=${INC}")
message(STATUS "ARCHS=${CMAKE_CUDA_ARCHITECTURES}")
"""


def test_consumer_of_the_tiny_cuda_nn_target_configures():
    cmake, nvcc, nl = shutil.which("cmake"), shutil.which("nvcc"), B.nlohmann_include_dir()
    if not (cmake and nvcc and nl):
        pytest.skip("needs cmake, nvcc and nlohmann/json.hpp")
    with tempfile.TemporaryDirectory() as tmp:
        with open(os.path.join(tmp, "CMakeLists.txt"), "w") as f:
            f.write(CONSUMER % (ROOT, os.path.join(ROOT, "tests", "cpp", "test_tcnn_headers.cu")))
        env = dict(os.environ, NLOHMANN_JSON_INCLUDE=nl)
        r = subprocess.run([cmake, "-S", tmp, "-B", os.path.join(tmp, "b"), "-DCMAKE_CUDA_COMPILER=" + nvcc], env=env,
                           capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "TCNN_DEFINITIONS=-DTCNN_MIN_GPU_ARCH=100" in r.stdout
    assert os.path.join(ROOT, "include") in r.stdout and nl in r.stdout
    assert "ARCHS=100a" in r.stdout
