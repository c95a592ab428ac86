"""``python setup.py install`` / ``pip install .`` - the install flow of the reference (its setup.py:20-42 drives
cmake; this one drives the in-tree ninja build of ``kraken_b200/_ext/_C.so`` for sm_100a) plus two console
commands with the names and flags of the reference's executables:

    scheduler_server --port 50000
    ps_server --port 50001 --addr 127.0.0.1:50001 --s_addr 127.0.0.1:50000 [--saved_dir DIR --max_save_count 3]
    kraken_zmq_frontend --s_addr 127.0.0.1:50000 --port 60000      (workers of the reference use these servers)

Working from the source tree needs none of this: ``python __graft_entry__.py`` builds in place.
"""
import os
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildWithNative(build_py):
    """Compiles the native extension into the package directory before the Python files are collected."""

    def run(self):
        sys.path.insert(0, HERE)
        from kraken_b200 import _build
        if not os.path.exists(_build.SO_PATH) or os.environ.get("KRAKEN_B200_REBUILD"):
            _build.build(verbose=True)
        super().run()


setup(
    name="kraken_b200",
    version="0.2.0",
    description="Blackwell-native sparse-embedding training framework with Kraken's API and checkpoint format",
    packages=find_packages(include=["kraken_b200", "kraken_b200.*"]),
    package_data={"kraken_b200": ["_ext/_C.so", "csrc/*.cc", "csrc/*/*.cc", "csrc/*/*.h", "csrc/*/*.cu", "csrc/*/*.cuh"]},
    python_requires=">=3.10",
    install_requires=["torch", "numpy"],
    cmdclass={"build_py": BuildWithNative},
    entry_points={"console_scripts": ["ps_server = kraken_b200.launch.ps_server:main",
                                      "scheduler_server = kraken_b200.launch.scheduler_server:main",
                                      "kraken_zmq_frontend = kraken_b200.runtime.zmq_frontend:main"]},
)
