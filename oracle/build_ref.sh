#!/usr/bin/env bash
# build_ref.sh -- TEST INFRASTRUCTURE.
#
# Compiles the UPSTREAM AdapTQ hot-path sources where they lie (the checkout
# named by the first argument, else by ADAPTQ_REFERENCE_DIR) into oracle/_ref/:
#
#   libadaptq_ref.so       -O3 -ffp-contract=off   parity build (bit-exact indices)
#   libadaptq_ref_fast.so  -O3 -mavx2 -mfma        timed CPU baseline build
#   libadaptq_ref_v2.so    -O3 -ffp-contract=off   upstream's second stack (RuntimeContext,
#                          SessionSnapshot, IKernelBackend) behind ref_v2_shim.cpp
#
# Nothing from upstream is copied into this repository; only object code lands
# in the git-ignored oracle/_ref/.  Upstream's own build system is not used.
#
# One-line fix: attention/attention.cpp:469-470 calls
#   vaccum1<BITS>(acc, vb + (size_t)s * pb, ..., cl, ch, padded)
# inside compute_avx2<K_BITS,V_BITS>, where BITS/pb/cl/ch do not exist (left
# over from before K and V got separate bit widths), so GCC rejects the file.
# The dense-V tail twenty lines above (:446) shows the intended call; the fix
# rewrites the two lines to match it.  It is applied on the fly through a pipe
# (the patched text is never written to disk) and the script refuses to build
# if the pre-image is not what it expects.
set -euo pipefail
REF="${1:-${ADAPTQ_REFERENCE_DIR:-}}"
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
if [ -z "$REF" ] || [ ! -f "$REF/attention/attention.cpp" ]; then
  echo "build_ref.sh: no upstream checkout given (argument or ADAPTQ_REFERENCE_DIR); keeping any prebuilt oracle/_ref" >&2
  exit 0
fi
mkdir -p "$OUT"

ATT="$REF/attention/attention.cpp"
grep -q 'vaccum1<BITS>(acc, vb + (size_t)s \* pb, w \* vscale\[s\] \* isp, cl, ch,' "$ATT" || {
  echo "build_ref.sh: attention.cpp does not contain the expected pre-image; refusing to patch" >&2
  exit 1
}
patched_attention() {
  sed -e 's/vaccum1<BITS>(acc, vb + (size_t)s \* pb, w \* vscale\[s\] \* isp, cl, ch,/vaccum1<V_BITS>(acc, vb + (size_t)s * v_pb, w * vscale[s] * isp, v_cl, v_ch,/' "$ATT"
}

SRCS=(core/fwht.cpp core/codebook.cpp core/quantizer.cpp core/adaptq_c_api.cpp
      core/adaptq_backend_vtable.cpp cache/ring_buffer.cpp kernels/scalar/kdot_scalar.cpp)
INC=(-I"$REF/include" -I"$REF/attention" -I"$REF/storage" -I"$REF/strategies" -I"$REF")

build_one() {  # $1 = output name, rest = flags
  local name="$1"; shift
  local tmp; tmp="$(mktemp -d)"
  for s in "${SRCS[@]}"; do
    g++ -std=c++17 -fPIC -fopenmp "$@" "${INC[@]}" -c "$REF/$s" -o "$tmp/$(basename "$s" .cpp).o"
  done
  # "../include/x.h" inside attention.cpp resolves through -I$REF/attention
  patched_attention | g++ -std=c++17 -fPIC -fopenmp "$@" "${INC[@]}" -x c++ -c - -o "$tmp/attention.o"
  g++ -std=c++17 -fPIC -fopenmp "$@" "${INC[@]}" -c "$HERE/ref_shim.cpp" -o "$tmp/ref_shim.o"
  g++ -shared -fopenmp -o "$OUT/$name" "$tmp"/*.o
  rm -f "$tmp"/*.o; rmdir "$tmp"
}

build_one libadaptq_ref.so -O3 -ffp-contract=off
build_one libadaptq_ref_fast.so -O3 -mavx2 -mfma

# Upstream's second stack.  Its strategies and storages are header-style sources that
# runtime/runtime_context.cpp includes itself (one translation unit, as upstream's own
# build does it), so only the files below are compiled; the AVX2 kernel file gets the
# machine flags upstream's build gives it.
V2_SRCS=(core/fwht.cpp core/codebook.cpp core/quantizer.cpp core/cost_optimizer.cpp core/quality_oracle.cpp
         kernels/scalar/kdot_scalar.cpp kernels/kernel_selector.cpp runtime/runtime_context.cpp
         replay/session_snapshot.cpp replay/replay_engine.cpp)
tmp="$(mktemp -d)"
for s in "${V2_SRCS[@]}"; do
  g++ -std=c++17 -fPIC -O3 -ffp-contract=off "${INC[@]}" -c "$REF/$s" -o "$tmp/$(basename "$s" .cpp).o"
done
g++ -std=c++17 -fPIC -O3 -mavx2 -mfma "${INC[@]}" -c "$REF/kernels/avx2/kdot_avx2.cpp" -o "$tmp/kdot_avx2.o"
g++ -std=c++17 -fPIC -O3 -ffp-contract=off "${INC[@]}" -c "$HERE/ref_v2_shim.cpp" -o "$tmp/ref_v2_shim.o"
g++ -shared -o "$OUT/libadaptq_ref_v2.so" "$tmp"/*.o
rm -f "$tmp"/*.o; rmdir "$tmp"
echo "built $OUT/libadaptq_ref.so, $OUT/libadaptq_ref_fast.so and $OUT/libadaptq_ref_v2.so"
