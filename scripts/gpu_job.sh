#!/usr/bin/env bash
# One parameterised runner for sessions on a GPU box: `scripts/gpu_job.sh <name> -- <command...>` runs the command from the
# repo root with its stdout/stderr captured under $GPU_JOB_OUT/<name>.log and the exit code in $GPU_JOB_OUT/<name>.rc.
# Several jobs can be chained in one session:  'scripts/gpu_job.sh a -- cmd1; scripts/gpu_job.sh b -- cmd2'
set -u
name="$1"; shift; [ "$1" = "--" ] && shift
out="${GPU_JOB_OUT:-gpurun_out}"; mkdir -p "$out"
export PYTHONPATH="$(pwd)${PYTHONPATH:+:$PYTHONPATH}"
( "$@" ) > "$out/${name}.log" 2>&1
rc=$?
echo "$rc" > "$out/${name}.rc"
echo "[gpu_job] ${name}: rc=${rc}"; tail -n 6 "$out/${name}.log"
exit 0
