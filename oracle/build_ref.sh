#!/bin/bash
# Builds, from the UNMODIFIED reference sources where they lie (nothing is copied into this repository), into oracle/_ref/:
#   libmlops_attention_ref.so  the reference FBLA library: its CUDA kernels compiled for sm_100 with nvcc directly (the
#                              reference's own build system refuses architectures newer than sm_90). The GPU parity
#                              tests and the bench's reference-GPU row load it next to the product library.
#   test_fbla_ours             the reference's own known-answer program (attention/fbla/tests/test_fbla.cu, public API
#                              only) linked against THIS repository's static library: the drop-in proof. Skipped when
#                              mlops_b200/lib/libmlops_attention.a has not been built yet.
# Test infrastructure only.   usage: oracle/build_ref.sh <path to the reference tree>   (default: $MLOPS_REFERENCE_ROOT)
set -euo pipefail
REF="${1:-${MLOPS_REFERENCE_ROOT:?give the path to the reference tree}}"
A="$REF/attention"
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
OURS="$HERE/../mlops_b200/lib/libmlops_attention.a"
[ -d "$A/fbla/src" ] || { echo "reference tree not found at $REF" >&2; exit 3; }
mkdir -p "$OUT/obj"
INC="-I$A/include -I$A/fbla/src -I$REF/positional/include -I$REF/positional/rope/src"
F="-O3 -std=c++17 -Xcompiler -ffp-contract=off,-fPIC -gencode arch=compute_100,code=sm_100 $INC"
if [ ! -f "$OUT/libmlops_attention_ref.so" ]; then
  nvcc $F -c -o "$OUT/obj/fbla.o" "$A/fbla/src/fbla.cu" &
  nvcc $F -DMLOPS_FBLA_CB=3 -DMLOPS_FBLA_FB=3 -c -o "$OUT/obj/fbla_inst_3p3.o" "$A/fbla/src/fbla_inst.cu" &
  nvcc $F -DMLOPS_FBLA_CB=4 -DMLOPS_FBLA_FB=2 -c -o "$OUT/obj/fbla_inst_4p2.o" "$A/fbla/src/fbla_inst.cu" &
  wait
  nvcc -shared -o "$OUT/libmlops_attention_ref.so" "$OUT/obj/fbla.o" "$OUT/obj/fbla_inst_3p3.o" "$OUT/obj/fbla_inst_4p2.o" -lcudart
fi
ls -la "$OUT/libmlops_attention_ref.so"
if [ -f "$OURS" ]; then
  nvcc -O2 -std=c++17 -gencode arch=compute_100a,code=sm_100a $INC -o "$OUT/test_fbla_ours" "$A/fbla/tests/test_fbla.cu" "$OURS"
  ls -la "$OUT/test_fbla_ours"
fi
