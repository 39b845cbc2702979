#!/usr/bin/env bash
# build_ref_binding.sh -- TEST INFRASTRUCTURE.
#
# Compiles UPSTREAM's own consumers of the C ABI, from the files where they lie
# in the upstream checkout (first argument, else ADAPTQ_REFERENCE_DIR), against
# THIS repository's libadaptq_b200.so, into the git-ignored oracle/_ref/:
#
#   adaptq_py<ext-suffix>.so    adapters/adapter_python.cpp +
#                               core/adaptq_backend_vtable.cpp, unchanged
#                               (upstream's pybind11 module; its Python package
#                               does `import adaptq_py`, adaptq/core.py:2-3)
#   adapter_standalone          adapters/adapter_standalone.c (plain-C program)
#   llamacpp_driver             adapters/adapter_llamacpp.cpp + llamacpp_driver.cpp
#                               (this directory: reads inputs, calls the adapter
#                               class, writes outputs)
#
# The two adapters still call the constructors with the argument list from before
# K and V got separate bit widths (7 arguments where the current declarations in
# upstream's own headers take 8: adapter_standalone.c:33-34 against
# include/adaptq.h:91-93, adapter_llamacpp.cpp:35 against
# include/adaptq_mha_backend.h:15), so neither compiles as shipped.  The missing
# v_bits argument is inserted on the fly through a pipe (nothing patched is
# written to disk); the script refuses to build them if the pre-image differs.
# Nothing from upstream is copied into this repository.
set -euo pipefail
REF="${1:-${ADAPTQ_REFERENCE_DIR:-}}"
HERE="$(cd "$(dirname "$0")" && pwd)"
ROOT="$(dirname "$HERE")"
OUT="$HERE/_ref"
LIBDIR="$ROOT/adaptq_b200"
if [ -z "$REF" ] || [ ! -f "$REF/adapters/adapter_python.cpp" ]; then
  echo "build_ref_binding.sh: no upstream checkout given (argument or ADAPTQ_REFERENCE_DIR); keeping any prebuilt oracle/_ref" >&2
  exit 0
fi
if [ ! -f "$LIBDIR/libadaptq_b200.so" ]; then
  echo "build_ref_binding.sh: $LIBDIR/libadaptq_b200.so is missing (python -m adaptq_b200.build)" >&2
  exit 1
fi
mkdir -p "$OUT"
PY="${PYTHON:-python3}"
PYINC="$("$PY" -m pybind11 --includes)"
SUFFIX="$("$PY" -c 'import sysconfig; print(sysconfig.get_config_var("EXT_SUFFIX"))')"
LINK=(-L"$LIBDIR" -l:libadaptq_b200.so -Wl,-rpath,'$ORIGIN/../../adaptq_b200')

# 1. the pybind11 module, sources unchanged
g++ -O2 -std=c++17 -shared -fPIC $PYINC -I"$REF/include" \
    "$REF/adapters/adapter_python.cpp" "$REF/core/adaptq_backend_vtable.cpp" \
    "${LINK[@]}" -o "$OUT/adaptq_py$SUFFIX"

# 2. the plain-C example program (v_bits inserted)
SA="$REF/adapters/adapter_standalone.c"
grep -q 'adaptq_mha_create(N_HEADS, HEAD_DIM, BITS, CAPACITY,' "$SA" || {
  echo "build_ref_binding.sh: adapter_standalone.c does not contain the expected pre-image" >&2; exit 1; }
sed -e 's/adaptq_mha_create(N_HEADS, HEAD_DIM, BITS, CAPACITY,/adaptq_mha_create(N_HEADS, HEAD_DIM, BITS, BITS, CAPACITY,/' "$SA" |
  gcc -O2 -I"$REF/adapters" -x c - "${LINK[@]}" -lm -o "$OUT/adapter_standalone"

# 3. the llama.cpp adapter class (v_bits inserted) behind a small driver
LC="$REF/adapters/adapter_llamacpp.cpp"
grep -q ': _backend(n_heads, head_dim, bits, capacity, seed, v_mass, hybrid_thresh)' "$LC" || {
  echo "build_ref_binding.sh: adapter_llamacpp.cpp does not contain the expected pre-image" >&2; exit 1; }
TMP="$(mktemp -d)"
sed -e 's/: _backend(n_heads, head_dim, bits, capacity, seed, v_mass, hybrid_thresh)/: _backend(n_heads, head_dim, bits, bits, capacity, seed, v_mass, hybrid_thresh)/' "$LC" |
  g++ -O2 -std=c++17 -I"$REF/adapters" -x c++ -c - -o "$TMP/adapter_llamacpp.o"
g++ -O2 -std=c++17 -I"$REF/adapters" -c "$HERE/llamacpp_driver.cpp" -o "$TMP/driver.o"
g++ "$TMP/driver.o" "$TMP/adapter_llamacpp.o" "${LINK[@]}" -o "$OUT/llamacpp_driver"
rm -f "$TMP"/*.o; rmdir "$TMP"
echo "built $OUT/adaptq_py$SUFFIX, $OUT/adapter_standalone and $OUT/llamacpp_driver against $LIBDIR/libadaptq_b200.so"
