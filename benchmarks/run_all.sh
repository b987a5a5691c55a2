#!/usr/bin/env bash
# Runs the single-GPU benchmarks one after another on the GPU that CUDA_VISIBLE_DEVICES names (default 0) and
# writes one log per benchmark. It only uses that GPU: it reserves no memory elsewhere, changes no clocks, power
# limits or modes, and starts nothing in the background (the reference's scripts/bench_isolated.sh pairs its runs
# with a process that occupies the other GPUs' memory; that part is deliberately absent).
#   benchmarks/run_all.sh [output-dir]
set -u
here="$(cd "$(dirname "$0")" && pwd)"
out="${1:-bench_logs}"
mkdir -p "$out"
export CUDA_VISIBLE_DEVICES="${CUDA_VISIBLE_DEVICES:-0}"
status=0
run() {
  name="$1"; shift
  echo "== $name: $*"
  if ! "$@" > "$out/$name.log" 2>&1; then
    rc=$?
    echo "   exit $rc (see $out/$name.log)"
    [ "$rc" -eq 77 ] || status=1
  fi
}
run kernel_cases    python "$here/kernel_cases.py" --case all --iters 10
run reference_bars  python "$here/reference_bars.py"
run serving         python "$here/bench_serving.py"
run moe             python "$here/bench_moe.py"
run decode_step     python "$here/bench_decode_step.py"
run cpu_decode_vnni python "$here/bench_cpu_decode_vnni.py"
run cpu             python "$here/bench_cpu.py"
run bench           python "$here/../bench.py"
exit $status
