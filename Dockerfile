# Build and test image for the B200 framework: CUDA 12.9 toolchain (nvcc cross-compiles sm_100a without
# a GPU), PyTorch with CUDA 12.8 wheels, the in-tree extension built at image build time.
#   docker build -t mythos-b200 .
#   docker run --gpus all --rm mythos-b200 python bench.py --steps 6 --warmup 3
FROM nvidia/cuda:12.9.1-devel-ubuntu24.04

ENV DEBIAN_FRONTEND=noninteractive PIP_BREAK_SYSTEM_PACKAGES=1 CUDA_HOME=/usr/local/cuda
RUN apt-get update && apt-get install -y --no-install-recommends \
        python3 python3-dev python3-pip g++ ninja-build git cmake && \
    rm -rf /var/lib/apt/lists/* && ln -sf /usr/bin/python3 /usr/local/bin/python

RUN pip install --no-cache-dir --index-url https://download.pytorch.org/whl/cu128 torch && \
    pip install --no-cache-dir numpy pytest pytest-timeout pybind11 ninja nvidia-ml-py fastapi uvicorn

WORKDIR /workspace/mythos_b200
COPY . .

# Compile every CUDA extension for sm_100a and the host library (no GPU needed), then the CPU test suite.
RUN python -c "import __graft_entry__ as g; g.build()" && \
    python -m pytest tests -x -q -m "not gpu"

CMD ["python", "-m", "pytest", "tests", "-x", "-q", "-m", "gpu"]
