#!/usr/bin/env bash
# Run a command while watching the kernel log for GPU faults; stop the command (by its own
# process group) on a hit.  Counterpart of the reference's step3b/run_guarded.sh:8-25, which
# greps `journalctl -k` on both laptops for Thunderbolt/driver fault patterns and docker-kills
# the benchmark containers.  Here the patterns are NVIDIA Xid / NVLink / fallen-off-the-bus
# messages and there is one host.  The command also runs under `timeout` (INNER_TO seconds), the
# same belt-and-braces the reference uses (step3b/node_launch.sh:28).
#   INNER_TO=600 POLL=3 ./run_guarded.sh torchrun --nproc-per-node 2 ... bench.py --gpus 2
set -uo pipefail
INNER_TO="${INNER_TO:-600}"; POLL="${POLL:-3}"
PAT="${PAT:-NVRM: Xid|NVLink.*(error|fatal)|fallen off the bus|GPU has fallen|blocked for more than}"
klog() { (journalctl -k --since "@$1" --no-pager 2>/dev/null || dmesg --since "@$1" 2>/dev/null || dmesg 2>/dev/null) | grep -E "$PAT" || true; }
START=$(date +%s)
setsid timeout -k 15 "$INNER_TO" "$@" &
PID=$!
PGID=$(ps -o pgid= "$PID" | tr -d ' ')
rc=0
while kill -0 "$PID" 2>/dev/null; do
  hit=$(klog "$START")
  if [ -n "$hit" ]; then
    echo "[guard] kernel log hit, stopping process group $PGID:" >&2
    echo "$hit" | tail -5 >&2
    kill -TERM -- "-$PGID" 2>/dev/null; sleep 5; kill -KILL -- "-$PGID" 2>/dev/null
    rc=99
    break
  fi
  sleep "$POLL"
done
wait "$PID" 2>/dev/null || rc=${rc:-$?}
[ "$rc" = 0 ] && wait "$PID" 2>/dev/null
exit "$rc"
