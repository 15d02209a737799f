# Runtime image: a CUDA 12.9 + PyTorch base with this repository and its kernels built for sm_100a.
# Build the kernels at image-build time (nvcc cross-compiles without a GPU):
#   docker build --build-arg BASE=<cuda-12.9 pytorch image> -t maxdiffusion_b200 .
ARG BASE=nvcr.io/nvidia/pytorch:25.06-py3
FROM ${BASE}
WORKDIR /workspace/maxdiffusion_b200
COPY . .
RUN bash setup.sh
ENV PYTHONPATH=/workspace/maxdiffusion_b200
ENTRYPOINT ["bash", "gpu_multi_process_run.sh"]
