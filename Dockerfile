# Training / evaluation image for dttt_b200 on B200 (sm_100a).  The code is mounted at run time
# (dttt_b200/tools/docker_run.sh); the image carries the toolchain and the Python environment only.
FROM nvidia/cuda:12.9.1-devel-ubuntu24.04

ENV DEBIAN_FRONTEND=noninteractive PIP_NO_CACHE_DIR=1 PYTHONUNBUFFERED=1
RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-pip python3-venv git ninja-build \
        libibverbs1 librdmacm1 ibverbs-providers && rm -rf /var/lib/apt/lists/*
RUN python3 -m venv /opt/venv
ENV PATH=/opt/venv/bin:${PATH}
RUN pip install "torch==2.11.*" --index-url https://download.pytorch.org/whl/cu128 && \
    pip install numpy pyarrow transformers sentencepiece pytest zstandard
# native kernels are built in-tree on first use (python -c "from dttt_b200 import build; build.build()")
WORKDIR /workspace
CMD ["bash"]
