#!/usr/bin/env bash
# Start / stop / inspect one qwserve instance.
#
#   ctl.sh start [qwserve arguments...]     e.g.  ctl.sh start --model-dir /models/qw --ple-dir /models/ples_fp8 --devices 0,1,2,3
#   ctl.sh stop | restart [args...] | status | logs | smoke
#   ctl.sh idle-stop [SECONDS=60]           stop the server once it has had nothing to do for that long (frees its GPUs)
#
# State lives in $QW_RUN_DIR (default: ./run next to this script): qwserve.pid, qwserve.log, qwserve.args.
# stop sends SIGTERM to the recorded pid only (the server drains its requests and gives the prefix cache time to flush),
# then waits up to $QW_STOP_SECONDS (default 60) before it reports failure; it never kills by name.
# (Role of the reference's server/ctl.sh.)
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
RUN="${QW_RUN_DIR:-$HERE/run}"
PIDFILE="$RUN/qwserve.pid"; LOG="$RUN/qwserve.log"; ARGS="$RUN/qwserve.args"
PY="${QW_PYTHON:-python}"
export PYTHONPATH="$HERE:$HERE/../..${PYTHONPATH:+:$PYTHONPATH}"

running() { [[ -f "$PIDFILE" ]] && kill -0 "$(cat "$PIDFILE")" 2>/dev/null; }

start() {
    mkdir -p "$RUN"
    if running; then echo "already running (pid $(cat "$PIDFILE"))"; return 0; fi
    if [[ $# -gt 0 ]]; then printf '%q ' "$@" > "$ARGS"; fi
    [[ -s "$ARGS" ]] || { echo "no arguments recorded: ctl.sh start --model-dir DIR ..." >&2; return 2; }
    # shellcheck disable=SC2046
    eval nohup "$PY" -m qwserve $(cat "$ARGS") >> "$LOG" 2>&1 &
    echo $! > "$PIDFILE"
    echo "started pid $(cat "$PIDFILE"), log $LOG"
}

stop() {
    running || { echo "not running"; rm -f "$PIDFILE"; return 0; }
    local pid; pid="$(cat "$PIDFILE")"
    kill -TERM "$pid"
    for _ in $(seq "${QW_STOP_SECONDS:-60}"); do
        kill -0 "$pid" 2>/dev/null || { rm -f "$PIDFILE"; echo "stopped"; return 0; }
        sleep 1
    done
    echo "pid $pid did not exit in ${QW_STOP_SECONDS:-60} s" >&2
    return 1
}

port() { grep -o -- '--port [0-9]*' "$ARGS" 2>/dev/null | awk '{print $2}' || true; }

case "${1:-}" in
    start) shift; start "$@" ;;
    stop) stop ;;
    restart) shift; stop; start "$@" ;;
    status) if running; then echo "running (pid $(cat "$PIDFILE"))"; else echo "stopped"; exit 3; fi ;;
    logs) tail -n "${2:-100}" "$LOG" ;;
    idle-stop) "$PY" -m qwserve.idle --url "http://127.0.0.1:$(p=$(port); echo "${p:-8000}")" --idle "${2:-60}" && stop ;;
    smoke) "$PY" -m qwserve.smoke --url "http://127.0.0.1:$(p=$(port); echo "${p:-8000}")" --follow-up ;;
    *) sed -n '2,13p' "${BASH_SOURCE[0]}"; exit 2 ;;
esac
