#!/bin/sh
# Builds libomoe.so for sm_100a next to the package (omega_ai_b200/libomoe.so).
# `build.sh check` builds the self-checking variant libomoe_check.so (-DOMOE_BOUNDS_CHECK, see check.cu) instead.
# Every .cu file is compiled on its own (in parallel, objects under build/, only when it or a header is
# newer than its object) and the objects are linked into one shared library.
set -e
cd "$(dirname "$0")"
NVCC=${NVCC:-/usr/local/cuda/bin/nvcc}
OUT=${OMOE_OUT:-../libomoe.so}
OBJDIR=${OMOE_OBJDIR:-build}
if [ "$1" = "check" ]; then
    OUT=../libomoe_check.so
    OBJDIR=build_check
    OMOE_NVCC_EXTRA="$OMOE_NVCC_EXTRA -DOMOE_BOUNDS_CHECK"
fi
FLAGS="-gencode arch=compute_100a,code=sm_100a -O3 -lineinfo -std=c++17 -Xcompiler -fPIC -Xcompiler -fvisibility=hidden ${OMOE_NVCC_EXTRA}"
SRCS="api.cu rmsnorm.cu router.cu route_small.cu permute.cu combine.cu experts_f32.cu experts_sm100.cu experts_sm100_splitk.cu experts_sm100_wgrad.cu backward.cu experts_decode.cu ep.cu check.cu"
mkdir -p "$OBJDIR"
# a changed flag set rebuilds everything
echo "$FLAGS" > "$OBJDIR/flags.new"
if ! cmp -s "$OBJDIR/flags.new" "$OBJDIR/flags" 2>/dev/null; then rm -f "$OBJDIR"/*.o; mv "$OBJDIR/flags.new" "$OBJDIR/flags"; fi
newest_hdr=$(ls -t *.cuh ../../include/omoe.h | head -1)
pids=""
for f in $SRCS; do
    o="$OBJDIR/${f%.cu}.o"
    if [ ! -f "$o" ] || [ "$f" -nt "$o" ] || [ "$newest_hdr" -nt "$o" ]; then
        $NVCC $FLAGS -c -o "$o" "$f" &
        pids="$pids $!"
    fi
done
for p in $pids; do wait "$p"; done
OBJS=""
for f in $SRCS; do OBJS="$OBJS $OBJDIR/${f%.cu}.o"; done
$NVCC -gencode arch=compute_100a,code=sm_100a -shared -cudart static -o "$OUT" $OBJS -ldl
