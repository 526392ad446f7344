"""Packaging: ``pip install .`` builds the sm_100a extension with nvcc and installs ``plexus_b200``
together with the reference-compatible ``plexus`` and ``performance`` import names.

The extension is built in-tree by ``plexus_b200.build_ext`` (direct nvcc, ``-gencode
arch=compute_100a,code=sm_100a``); no GPU is needed at build time.  Set ``PLEXUS_SKIP_BUILD=1`` to
install the Python sources only (CPU use: gloo ranks, data pipeline, cost models).
"""

import os
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


class BuildWithKernels(build_py):
    def run(self):
        if os.environ.get("PLEXUS_SKIP_BUILD", "0") in ("", "0"):
            sys.path.insert(0, ROOT)
            from plexus_b200 import build_ext

            build_ext.build(force=False, verbose=True)
        super().run()


setup(
    name="plexus-b200",
    version="0.1.0",
    description="3D-parallel full-graph GCN training for NVIDIA B200 (sm_100a): hand-written CUDA kernels, "
                "peer-memory collectives over NVLink, the API of hpcgroup/plexus",
    packages=find_packages(include=["plexus_b200", "plexus_b200.*", "plexus", "plexus.*", "performance"]),
    package_data={"plexus_b200": ["_C.so", "csrc/*.cpp", "csrc/include/*", "csrc/kernels/*.cu", "perf/*.json"]},
    python_requires=">=3.10",
    install_requires=["torch>=2.5", "numpy"],
    extras_require={"mtx": ["scipy"]},
    cmdclass={"build_py": BuildWithKernels},
)
