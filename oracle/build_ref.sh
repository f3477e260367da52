#!/bin/bash
# Builds the UNMODIFIED reference FBLA library (its CUDA kernels, compiled for sm_100 with nvcc directly, not through the
# reference's own build system, which refuses architectures newer than sm_90) into oracle/_ref/ as a shared object.
# Test infrastructure: the GPU parity tests and the bench's reference-GPU row load it next to the product library to
# compare results on identical inputs. Sources are compiled where they lie; nothing is copied into this repository.
#   usage: oracle/build_ref.sh <path to the reference tree>   (default: $MLOPS_REFERENCE_ROOT)
set -euo pipefail
REF="${1:-${MLOPS_REFERENCE_ROOT:?give the path to the reference tree}}"
A="$REF/attention"
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
[ -d "$A/fbla/src" ] || { echo "reference tree not found at $REF" >&2; exit 3; }
mkdir -p "$OUT/obj"
F="-O3 -std=c++17 -Xcompiler -ffp-contract=off,-fPIC -gencode arch=compute_100,code=sm_100 -I$A/include -I$A/fbla/src -I$REF/positional/include -I$REF/positional/rope/src"
nvcc $F -c -o "$OUT/obj/fbla.o" "$A/fbla/src/fbla.cu" &
nvcc $F -DMLOPS_FBLA_CB=3 -DMLOPS_FBLA_FB=3 -c -o "$OUT/obj/fbla_inst_3p3.o" "$A/fbla/src/fbla_inst.cu" &
nvcc $F -DMLOPS_FBLA_CB=4 -DMLOPS_FBLA_FB=2 -c -o "$OUT/obj/fbla_inst_4p2.o" "$A/fbla/src/fbla_inst.cu" &
wait
nvcc -shared -o "$OUT/libmlops_attention_ref.so" "$OUT/obj/fbla.o" "$OUT/obj/fbla_inst_3p3.o" "$OUT/obj/fbla_inst_4p2.o" -lcudart
ls -la "$OUT/libmlops_attention_ref.so"
