# Build and run image for penny-b200 on a B200 (sm_100a) box.
#
# Unlike the reference's image (Dockerfile:1-83: CUDA 12.9.1 + InfiniBand/RDMA userland + the
# nvshmem-cuda-12 package + nsight-systems) this one needs no NVSHMEM and no RDMA stack: the
# library talks to peer GPUs through CUDA VMM / IPC mappings and the NVSwitch multicast
# object, all of which come with the CUDA driver.
#
#   docker build -t penny-b200 .
#   docker run --gpus all --ipc=host --shm-size=8g --ulimit memlock=-1 penny-b200 \
#       torchrun --nproc-per-node 8 extra/benchmark_allreduce.py
#
# --ipc=host (or a large --shm-size): the ranks pass POSIX file descriptors of their heap
# allocations over Unix sockets and torch.distributed uses shared memory for gloo.
FROM nvidia/cuda:12.9.1-cudnn-devel-ubuntu22.04

ENV DEBIAN_FRONTEND=noninteractive \
    PIP_NO_CACHE_DIR=1 \
    TORCH_CUDA_ARCH_LIST=10.0a \
    MAX_JOBS=16

RUN apt-get update && apt-get install -y --no-install-recommends \
        python3 python3-dev python3-pip python3-venv git build-essential ninja-build gdb \
    && rm -rf /var/lib/apt/lists/* \
    && ln -sf /usr/bin/python3 /usr/bin/python

# PyTorch built against CUDA 12.8+ knows sm_100; NCCL comes bundled and is only used as the
# baseline in the benchmarks and by torch.distributed for the bootstrap broadcast.
RUN python -m pip install --upgrade pip setuptools wheel \
    && python -m pip install torch --index-url https://download.pytorch.org/whl/cu128 \
    && python -m pip install numpy pytest pybind11 nvidia-ml-py

WORKDIR /workspace/penny-b200
COPY . .

# nvcc cross-compiles for sm_100a without a GPU, so the extension (and the host protocol
# simulator) are built at image build time; the CPU test tier runs here as a smoke check.
RUN python setup.py build_ext --inplace \
    && python -m pytest tests -q -m "not gpu" -x

ENV PYTHONPATH=/workspace/penny-b200
CMD ["python", "-m", "pytest", "tests", "-q", "-m", "gpu"]
