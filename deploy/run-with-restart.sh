#!/usr/bin/env bash
# Restart loop with a crash window: gives up when the server dies more than MAX_CRASHES times
# within WINDOW_S seconds (same policy as the reference's deploy/run-with-restart.sh:28-56).
set -u
MAX_CRASHES=${MAX_CRASHES:-5}
WINDOW_S=${WINDOW_S:-300}
crashes=()
while true; do
  python3 -m hartsyinference_b200.cli serve "$@"
  code=$?
  [ "$code" -eq 0 ] && exit 0
  now=$(date +%s)
  crashes+=("$now")
  recent=()
  for t in "${crashes[@]}"; do [ $((now - t)) -le "$WINDOW_S" ] && recent+=("$t"); done
  crashes=("${recent[@]}")
  if [ "${#crashes[@]}" -gt "$MAX_CRASHES" ]; then
    echo "server crashed ${#crashes[@]} times within ${WINDOW_S}s; giving up" >&2
    exit "$code"
  fi
  echo "server exited with $code; restarting in 3s" >&2
  sleep 3
done
