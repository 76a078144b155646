#!/usr/bin/env bash
# Builds the UNMODIFIED reference CUDA kernel pack (packs/cuda/pack.cu, a single
# translation unit) from a read-only checkout of truespar/paddock into
# oracle/_ref/pd-cuda-ref.so.  Test infrastructure only: the resulting library
# is a second, independent checker (the reference's own GPU results for the
# same C-ABI slots).  Nothing in the product links, loads or calls it.
#
#   oracle/build_ref.sh [/path/to/paddock]     (default: $PADDOCK_REFERENCE, else the checkout
#                                               mounted next to the repository)
#
# Flags follow the reference's packs/cuda/build.sh for an arch list of "100":
# plain sm_100 + the sm_100a feature target, PD_TC5_HOST and PD_BS_HOST.
set -euo pipefail
here="$(cd "$(dirname "$0")" && pwd)"
ref="${1:-${PADDOCK_REFERENCE:-$(cd "$here/../.." && pwd)/reference}}"
src="$ref/packs/cuda/pack.cu"
out="$here/_ref/pd-cuda-ref.so"
[ -f "$src" ] || { echo "reference checkout not found at $ref: skipping"; exit 0; }
# the slot list the ABI tests pin the header against
python "$here/../tests/golden/gen_kernel_table.py" "$ref"
mkdir -p "$here/_ref"
if [ -f "$out" ] && [ "$out" -nt "$src" ]; then
    echo "up to date: $out"; exit 0
fi
nvcc -O3 --threads "${PD_BUILD_THREADS:-2}" \
    -gencode=arch=compute_100,code=sm_100 \
    -gencode=arch=compute_100a,code=sm_100a \
    -DPD_TC5_HOST=1 -DPD_BS_HOST=1 \
    -Xcompiler -fPIC --shared -o "$out.tmp" "$src"
mv "$out.tmp" "$out"
echo "built: $out"
