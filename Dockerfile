# Image for one 8-GPU B200 node.  The base image must provide CUDA 12.8+ (nvcc for sm_100a) and PyTorch 2.8+ with NCCL;
# nothing is downloaded at build time except what the base image's package index offers.
ARG BASE=nvcr.io/nvidia/pytorch:25.06-py3
FROM ${BASE}
WORKDIR /opt/aspec-b200
COPY pyproject.toml README.md ./
COPY aspec_b200 ./aspec_b200
COPY tools ./tools
COPY examples ./examples
# pure-Python install of the package with its sources, then the in-place build of the kernel and runtime libraries
RUN python -m pip install --no-deps --no-build-isolation -e . \
 && python -m aspec_b200.build
ENV NCCL_NVLS_ENABLE=1
ENTRYPOINT ["aspec-b200"]
CMD ["doctor"]
