#!/bin/bash
# Build the image (kernels are compiled for sm_100a at build time) and open a shell with all GPUs, host IPC and
# unlimited locked memory (NCCL and the symmetric-memory rendezvous need both).
set -x
ROOT=$(cd "$(dirname "$0")/../.." && pwd)
docker build -t openrlhf_b200:latest -f "$ROOT/dockerfile/Dockerfile" "$ROOT"
docker run --rm -it --gpus all --ipc=host --ulimit memlock=-1 --ulimit stack=67108864 \
   -v "$ROOT/ckpt:/opt/openrlhf_b200/ckpt" openrlhf_b200:latest bash
