#!/usr/bin/env bash
# One-shot launcher for the vLLM TP benchmark on this host (all ranks local; the reference's
# run_vllm_tp.sh / node_launch.sh start one docker container per laptop over ssh instead).
# MODE picks the all-reduce under test, like the reference's NCCL transport modes
# (step3b/node_launch.sh:12-18: gdr / hostbounce / socket / sockettb):
#   tbvcoll | nccl (NVLink P2P, NVLS if available) | nccl-timed | nccl-hostbounce (P2P off: through host shared
#   memory) | nccl-socket (P2P and shared memory off: loopback sockets)
#   TP=2 BATCH=8 OUT=128 MODE=tbvcoll ROUNDS=3 INNER_TO=900 ./run_vllm_tp.sh [--synth llama3-8b | --model DIR]
set -euo pipefail
TP="${TP:-2}"; BATCH="${BATCH:-8}"; OUT="${OUT:-128}"; MODE="${MODE:-tbvcoll}"; ROUNDS="${ROUNDS:-3}"
INNER_TO="${INNER_TO:-900}"; PORT="${PORT:-29640}"
EXTRA=()
case "$MODE" in
  tbvcoll) EXTRA+=(--tbvcoll) ; [ "${TBVEAGER:-0}" = 1 ] && EXTRA+=(--tbv-eager) ;;
  nccl) ;;
  nccl-timed) EXTRA+=(--time-nccl) ;;
  nccl-hostbounce) export NCCL_P2P_DISABLE=1 NCCL_NVLS_ENABLE=0 ;;
  nccl-socket) export NCCL_P2P_DISABLE=1 NCCL_SHM_DISABLE=1 NCCL_NVLS_ENABLE=0 NCCL_SOCKET_IFNAME=lo ;;
  *) echo "MODE must be tbvcoll | nccl | nccl-timed | nccl-hostbounce | nccl-socket" >&2; exit 2 ;;
esac
exec timeout -k 15 "$INNER_TO" python -m torch.distributed.run --nnodes=1 --nproc-per-node "$TP" --master-addr 127.0.0.1 \
  --master-port "$PORT" -m libtbvcoll_b200.integrations.vllm_tp_bench --tp "$TP" --batch "$BATCH" --out-tokens "$OUT" \
  --rounds "$ROUNDS" "${EXTRA[@]}" "$@"
