#!/bin/sh
# Regenerates the PTX fixture of tests/test_gpu_generated_blocks.py::test_ptx_image_path.
set -e
cd "$(dirname "$0")"
/usr/local/cuda/bin/nvcc -ptx -arch=compute_100a -o scale_block_sm100a.ptx scale_block.cu
