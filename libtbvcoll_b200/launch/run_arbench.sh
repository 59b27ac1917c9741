#!/usr/bin/env bash
# Run the native all-reduce microbenchmark on N GPUs of this host, one process per GPU.
# Counterpart of the reference's run_ar2.sh / run_armr.sh (build, start rank 0, start the
# other ranks), minus docker and ssh: all ranks are local.  Every rank runs under `timeout`
# so that a stuck rank can never hold a GPU (the reference wraps its runs the same way,
# step4/run_tbvcoll.sh:9-10).
#   WORLD=2 BYTES=57344 ITERS=2000 PORT=18990 INNER_TO=120 ./run_arbench.sh
set -euo pipefail
HERE="$(cd "$(dirname "$0")/.." && pwd)"
WORLD="${WORLD:-2}"; BYTES="${BYTES:-57344}"; ITERS="${ITERS:-2000}"; PORT="${PORT:-18990}"; INNER_TO="${INNER_TO:-120}"
python -m libtbvcoll_b200._build >/dev/null
pids=()
for ((r = WORLD - 1; r >= 0; r--)); do
  timeout -k 5 "$INNER_TO" "$HERE/tbv_arbench" "$r" "$WORLD" "$r" "$BYTES" "$ITERS" 127.0.0.1 "$PORT" &
  pids+=($!)
done
rc=0
for p in "${pids[@]}"; do wait "$p" || rc=$?; done
exit $rc
