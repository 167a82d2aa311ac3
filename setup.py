from setuptools import find_packages, setup

setup(
    name="lm-engine",
    version="0.0.1.dev0",
    description="LLM training engine for NVIDIA B200 (tcgen05 kernels, NVLink peer-memory collectives)",
    packages=find_packages(include=["lm_engine", "lm_engine.*"]),
    python_requires=">=3.10",
    install_requires=open("requirements.txt").read().split(),
)
