#!/usr/bin/env bash
# TEST INFRASTRUCTURE ONLY.
#
# Compiles the reference project's own KV-cache / paged-attention translation units,
# unmodified and from where they lie in the reference checkout, into
# oracle/_ref/libwarp34_ref.so.  The flags are the reference build's own
# (crates/warp34-kernels/build.rs:52-59: -O3 -lineinfo -std=c++17 --expt-relaxed-constexpr
# -use_fast_math -extended-lambda) with the architecture switched to sm_100a.
# Nothing from the reference is copied into this repository; only the built library
# lands in oracle/_ref/, which is git-ignored.
#
# The library is the bit-exactness checker for the TQ4 append path and the
# dequant-then-attend checker for attention.  op_norms_rope_act.cu (the layer's QK-norm / RoPE
# producer and its output-gate kernels) is built in as the checker of the fused producer and of
# the output epilogue, op_qsa.cu (query-sparse attention over selected 4-token groups) as the checker of
# the sparse attention entry points.  The product never links or loads it.
#
# usage: oracle/build_ref.sh [reference_root]      (default: $WARP34_REFERENCE_ROOT, else the checkout next to this repository)
set -euo pipefail
REF="${1:-${WARP34_REFERENCE_ROOT:-$(cd "$(dirname "$0")/../.." && pwd)/reference}}"
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
CSRC="$REF/crates/warp34-kernels/csrc"
VENDOR="$REF/crates/warp34-kernels/vendor/vision-fa2"
NVCC="${NVCC:-nvcc}"
if [ ! -d "$CSRC" ]; then
  echo "reference sources not found at $CSRC; keeping any prebuilt $OUT" >&2
  exit 0
fi
mkdir -p "$OUT/obj"
FLAGS="-gencode arch=compute_100a,code=sm_100a -O3 -lineinfo -std=c++17 --expt-relaxed-constexpr -use_fast_math -extended-lambda -Xcompiler -fPIC -I $CSRC"
FA2_FLAGS="-I $VENDOR/flash-attn/src -I $VENDOR/flash-attn/stubs -I $VENDOR/cutlass/include -include $VENDOR/flash-attn/fa2_compat_prelude.h -DFLASHATTENTION_DISABLE_DROPOUT -DFLASHATTENTION_DISABLE_ALIBI -DFLASHATTENTION_DISABLE_SOFTCAP -DFLASHATTENTION_DISABLE_LOCAL"
pids=()
for stem in op_kv_cache op_paged_attn op_init op_norms_rope_act op_qsa; do
  if [ "$OUT/obj/$stem.o" -nt "$CSRC/ops/$stem.cu" ]; then continue; fi
  $NVCC $FLAGS -c "$CSRC/ops/$stem.cu" -o "$OUT/obj/$stem.o" &
  pids+=($!)
done
if [ ! "$OUT/obj/op_paged_fa2.o" -nt "$CSRC/ops/op_paged_fa2.cu" ]; then
  $NVCC $FLAGS $FA2_FLAGS -c "$CSRC/ops/op_paged_fa2.cu" -o "$OUT/obj/op_paged_fa2.o" &
  pids+=($!)
fi
for p in "${pids[@]}"; do wait "$p"; done
${CC:-gcc} -O2 -fPIC -c "$HERE/ref_link_stubs.c" -o "$OUT/obj/ref_link_stubs.o"
$NVCC -shared -o "$OUT/libwarp34_ref.so" "$OUT"/obj/ref_link_stubs.o "$OUT"/obj/op_kv_cache.o "$OUT"/obj/op_paged_attn.o \
  "$OUT"/obj/op_init.o "$OUT"/obj/op_paged_fa2.o "$OUT"/obj/op_norms_rope_act.o "$OUT"/obj/op_qsa.o -lcublas -lcublasLt -lcudart
echo "built $OUT/libwarp34_ref.so"
