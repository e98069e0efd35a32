# Build image for cubework_b200: CUDA 12.9 toolchain (nvcc cross-compiles sm_100a without a GPU) + PyTorch.
FROM nvcr.io/nvidia/pytorch:25.06-py3

WORKDIR /workspace/cubework_b200
COPY . .
RUN pip install --no-cache-dir --no-build-isolation -e . && python -m cubework_b200.ops.build
