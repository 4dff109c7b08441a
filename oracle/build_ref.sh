#!/usr/bin/env bash
# Builds oracle/_ref/libraft_ref.so: the reference's OWN raft::linalg reduction kernels, compiled
# for sm_100a from the headers where they lie in the reference checkout (never copied), behind
# the small C ABI of oracle/ref_*.cu. Test infrastructure: used to validate the CPU oracle and
# as the "reference" column of the benchmark.
#
#   oracle/build_ref.sh [path of the reference checkout; default: $RAFT_REFERENCE_DIR, else a directory
#                        named `reference` beside this repository]
#
# The reference's cmake build cannot configure offline (it fetches rapids-cmake, rmm,
# rapids_logger, gtest), but this path is header-only; it needs
#   - four stand-in headers for rmm / rapids_logger (oracle/ref_shim/), and
#   - a CCCL new enough for cuda/std mdspan concepts: the copy bundled with flashinfer.
# Exits 0 without building when the reference checkout or that CCCL is absent.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${1:-${RAFT_REFERENCE_DIR:-$HERE/../../reference}}"
OUT="$HERE/_ref"
CCCL="$(python - <<'PY'
import importlib.util, os
spec = importlib.util.find_spec("flashinfer")
print(os.path.join(os.path.dirname(spec.origin), "data", "cccl") if spec and spec.origin else "")
PY
)"
if [ ! -d "$REF/cpp/include/raft" ]; then echo "build_ref: no reference checkout at $REF - skipped"; exit 0; fi
if [ -z "$CCCL" ] || [ ! -d "$CCCL/libcudacxx/include" ]; then echo "build_ref: no recent CCCL found - skipped"; exit 0; fi
mkdir -p "$OUT"
FLAGS=(-std=c++20 --expt-extended-lambda --expt-relaxed-constexpr -gencode arch=compute_100a,code=sm_100a -O3
       -lineinfo -Xcompiler -fPIC,-fvisibility=hidden -w
       -I"$HERE/ref_shim" -I"$CCCL/libcudacxx/include" -I"$CCCL/cub" -I"$CCCL/thrust"
       -I"$REF/cpp/include" -I"$HERE/../include")
pids=()
TUS=(ref_reduce_rows ref_reduce_cols ref_bykey_kvp ref_normalize ref_map_reduce)
for tu in "${TUS[@]}"; do
  if [ "$OUT/$tu.o" -nt "$HERE/$tu.cu" ] && [ "$OUT/$tu.o" -nt "$HERE/ref_common.cuh" ]; then continue; fi
  nvcc "${FLAGS[@]}" -c "$HERE/$tu.cu" -o "$OUT/$tu.o" &
  pids+=($!)
done
for p in "${pids[@]:-}"; do [ -n "$p" ] && wait "$p"; done
OBJS=()
for tu in "${TUS[@]}"; do OBJS+=("$OUT/$tu.o"); done
nvcc -gencode arch=compute_100a,code=sm_100a -shared -o "$OUT/libraft_ref.so" "${OBJS[@]}"
echo "build_ref: built $OUT/libraft_ref.so"
