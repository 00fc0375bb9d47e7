# Serving image for one 8 x B200 box (sm_100a only).  Counterpart of the reference's container recipe; the kernels
# are compiled in-tree at build time, the entry point is the OpenAI / Anthropic compatible server.
#
#   docker build -t ninfer-fusion-b200 .
#   docker run --gpus all --ipc=host -p 8000:8000 -v /models:/models ninfer-fusion-b200 \
#       --artifact /models/model.ninfer --host 0.0.0.0 --port 8000
#   (tensor parallel: add `--tp 8`; the container then starts one rank per GPU through torch.distributed.run)
FROM nvidia/cuda:12.9.1-devel-ubuntu24.04

ENV DEBIAN_FRONTEND=noninteractive PIP_NO_CACHE_DIR=1 PYTHONUNBUFFERED=1
RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-pip python3-venv ninja-build g++ \
    && rm -rf /var/lib/apt/lists/*
RUN python3 -m venv /opt/venv
ENV PATH=/opt/venv/bin:$PATH
RUN pip install "torch==2.11.*" --index-url https://download.pytorch.org/whl/cu128 \
    && pip install numpy pybind11 ninja pytest

WORKDIR /opt/ninfer-fusion-b200
COPY . .
# nvcc cross-compiles for sm_100a without a GPU in the build container
RUN python -m ninfer_fusion_b200._build && python -m pytest tests -q -m "not gpu" -x -k "artifact or frontend or hostdiag"

EXPOSE 8000
ENTRYPOINT ["python", "-m", "ninfer_fusion_b200.cli", "serve"]
CMD ["--help"]
