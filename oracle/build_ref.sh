#!/bin/sh
# Compiles the reference's own generated C artefacts from where they lie in the reference tree
# into oracle/_ref/ (git-ignored outputs only; no reference source is copied into this repo).
#   usage: oracle/build_ref.sh [REFERENCE_ROOT]        (default: $DGEN_REFERENCE_ROOT, else a checkout named
#                                                       "reference" beside this repository; absent = skip)
# The reference runtime header is written for AArch64; the single ARM-only inline-asm register
# constraint ("+w", a NEON register) is rewritten to the x86 vector-register constraint ("+x")
# in a generated copy under _ref/include, and <arm_neon.h> resolves to oracle/neon_shim.
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
REF="${1:-${DGEN_REFERENCE_ROOT:-$HERE/../../reference}}"
OUT="$HERE/_ref"
SRC="$REF/toolchain/generated/hermetic"
[ -d "$SRC" ] || { echo "build_ref: $SRC not found; skipping" >&2; exit 0; }
mkdir -p "$OUT/include"
sed 's/"+w"(bits)/"+x"(bits)/' "$REF/toolchain/include/dgen_runtime.h" > "$OUT/include/dgen_runtime.h"
for name in scalar-synth feedback-delay-effect wavetable-instrument spectral-effect; do
  gcc -O2 -std=gnu11 -fPIC -shared -w -fno-fast-math -ffp-contract=off -fno-builtin \
      -I"$OUT/include" -I"$HERE/neon_shim" -o "$OUT/$name.so" "$SRC/$name.c" -lm
done
gcc -O2 -std=gnu11 -fPIC -shared -o "$OUT/libref_harness.so" "$HERE/ref_harness.c" -ldl -lm
echo "build_ref: built $(ls "$OUT"/*.so | wc -l) objects in $OUT"
