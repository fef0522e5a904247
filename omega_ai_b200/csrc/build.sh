#!/bin/sh
# Builds libomoe.so for sm_100a next to the package (omega_ai_b200/libomoe.so).
set -e
cd "$(dirname "$0")"
NVCC=${NVCC:-/usr/local/cuda/bin/nvcc}
$NVCC -gencode arch=compute_100a,code=sm_100a -O3 -lineinfo -std=c++17 \
    -Xcompiler -fPIC -Xcompiler -fvisibility=hidden -shared -cudart static \
    ${OMOE_NVCC_EXTRA} \
    -o ${OMOE_OUT:-../libomoe.so} api.cu rmsnorm.cu router.cu route_small.cu permute.cu combine.cu experts_f32.cu experts_sm100.cu experts_sm100_pair.cu experts_sm100_splitk.cu experts_sm100_wgrad.cu backward.cu experts_decode.cu ep.cu \
    -ldl
