#!/usr/bin/env bash
# TEST INFRASTRUCTURE. Builds oracle/_ref/libbm_ref.so: the reference's unmodified C11 host code
# (read in place from the reference checkout, never copied into this repository's history) linked
# against oracle/ref_cpu_backend.cpp, which runs the reference's Metal kernel sources on CPU.
#
# The only edit applied to a reference source is made on a generated copy under oracle/_ref/staged/:
# the two per-thread array bounds of the whole-row attention kernels (ATTN_MAXS_FWD in
# src/kernels/forward.metal:1810 and ATTN_MAXS in src/kernels/backward.metal:664, both 256) are raised
# so the same kernels can serve as the oracle for sequences longer than 256 tokens.
#
# usage: oracle/build_ref.sh [reference_dir]      (default: $BM_REFERENCE, else a directory named "reference" beside this repository)
set -euo pipefail
HERE="$(cd "$(dirname "$0")" && pwd)"
REF="${1:-${BM_REFERENCE:-$HERE/../../reference}}"
OUT="$HERE/_ref"
MAXS="${BM_REF_ATTN_MAXS:-8192}"
if [ ! -f "$REF/src/baremetal/trainer.c" ]; then
  echo "build_ref: no reference checkout at $REF" >&2
  exit 3
fi
mkdir -p "$OUT/staged" "$OUT/obj"
sed "s/^#define ATTN_MAXS_FWD 256/#define ATTN_MAXS_FWD $MAXS/" "$REF/src/kernels/forward.metal" > "$OUT/staged/forward.metal"
sed "s/^#define ATTN_MAXS 256/#define ATTN_MAXS $MAXS/" "$REF/src/kernels/backward.metal" > "$OUT/staged/backward.metal"
grep -q "ATTN_MAXS_FWD $MAXS" "$OUT/staged/forward.metal"
grep -q "ATTN_MAXS $MAXS" "$OUT/staged/backward.metal"

CFLAGS="-std=c11 -D_GNU_SOURCE -DBAREMETAL_TRAIN -D__fp16=_Float16 -O2 -fPIC -w -I$REF/include -I$REF/src"
objs=()
for f in "$REF"/src/baremetal/*.c "$REF/src/kernels/registry.c" "$REF/src/utils/log.c" "$REF/tools/run.c" "$HERE/ref_shim.c"; do
  o="$OUT/obj/$(basename "${f%.c}").o"
  gcc $CFLAGS -c "$f" -o "$o"
  objs+=("$o")
done
g++ -std=c++17 -O2 -fPIC -fopenmp -ffp-contract=off -D__HAVE_BFLOAT__=1 -Wno-attributes -w \
  -I"$HERE/metal_stub" -I"$REF/include" -I"$REF/src" \
  -DBM_REF_FORWARD_METAL="\"$OUT/staged/forward.metal\"" \
  -DBM_REF_BACKWARD_METAL="\"$OUT/staged/backward.metal\"" \
  -DBM_REF_ADAMW_METAL="\"$REF/src/anneal/adamw.metal\"" \
  -c "$HERE/ref_cpu_backend.cpp" -o "$OUT/obj/ref_cpu_backend.o"
g++ -shared -fopenmp -Wl,--no-undefined -o "$OUT/libbm_ref.so" "${objs[@]}" "$OUT/obj/ref_cpu_backend.o" -lm
echo "built $OUT/libbm_ref.so"

# The same unmodified reference host objects linked against the product's CUDA backend (its backend_* functions, include/backend.h)
# instead of the CPU backend above, and the reference's own kernel test programs built against that backend. Both are checkers for
# the backend ABI of the product; they need a GPU to run.
PKG="$HERE/../bare.metal_b200"
if [ -f "$PKG/libbaremetal_b200.so" ]; then
  gcc -shared -Wl,-Bsymbolic -Wl,--no-undefined -o "$OUT/libbm_ref_cuda.so" "${objs[@]}" -L"$PKG" -lbaremetal_b200 \
    -Wl,-rpath,'$ORIGIN/../../bare.metal_b200' -lm
  echo "built $OUT/libbm_ref_cuda.so"
  mkdir -p "$OUT/kernel_tests"
  for t in matmul_bwd_test rmsnorm_bwd_test rope_seq_bwd_test rope_real_test xent_bwd_test embed_bwd_test adamw_test attn_bwd_test \
           attn_fwd_test attn_real_test train_attn_tiled_test; do
    gcc $CFLAGS -o "$OUT/kernel_tests/$t" "$REF/test/$t.c" "$OUT/obj/log.o" -L"$PKG" -lbaremetal_b200 \
      -Wl,-rpath,'$ORIGIN/../../../bare.metal_b200' -lm
  done
  echo "built $OUT/kernel_tests/"
fi
