"""Packaging: builds the CUDA library in-tree and registers the vLLM plugin entry points
(the reference registers ``vllm.platform_plugins`` and ``vllm.general_plugins`` the same way,
setup.py:325-358 of vllm-gcu)."""
from setuptools import find_packages, setup
from setuptools.command.build_py import build_py


class BuildWithKernels(build_py):
    def run(self):
        from vllm_gcu_b200.csrc.build import build
        build()                      # nvcc -gencode arch=compute_100a,code=sm_100a, one .so
        from vllm_gcu_b200.utils.shm_ring import build_host_library
        build_host_library()         # g++: host-only library (shared-memory command ring)
        super().run()


setup(
    name="vllm_gcu_b200",
    version="0.1.0",
    description="Blackwell-native LLM serving framework with the capabilities of vllm-gcu",
    # the benchmark tools install as ``vllm_utils`` (``python -m vllm_utils.benchmark_serving``),
    # the name the reference's tools are installed under
    packages=find_packages(include=["vllm_gcu_b200", "vllm_gcu_b200.*"]) + [
        "vllm_utils", "vllm_utils.kernels", "vllm_utils.evaluate_datasets",
        "vllm_utils.disagg_benchmarks"],
    package_dir={"vllm_utils": "benchmarks"},
    package_data={"vllm_gcu_b200": ["_b200.so", "_b200_host.so", "csrc/*.cu", "csrc/*.cuh",
                                    "csrc/*.h", "csrc/host/*.cpp"]},
    python_requires=">=3.10",
    install_requires=["torch", "numpy"],
    extras_require={"server": ["fastapi", "uvicorn"], "kv": ["pyzmq", "msgpack"]},
    cmdclass={"build_py": BuildWithKernels},
    entry_points={
        "vllm.platform_plugins": ["b200 = vllm_gcu_b200:register_platform_plugins"],
        "vllm.general_plugins": ["b200_models = vllm_gcu_b200:register_custom_models"],
        "console_scripts": [
            "vllm-b200-server = vllm_gcu_b200.entrypoints.api_server:main",
            "vllm-b200-router = vllm_utils.router:main",
        ],
    },
)
