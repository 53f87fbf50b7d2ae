#!/bin/sh
# Runs the prebuilt reference programs of baseline/_ref once each (their own timing loops) and
# this library's driver on the same workloads; prints every timing line.
here=$(dirname "$0")
for p in center_gemv_topk gemv_topk baseline_1; do
  if [ -x "$here/_ref/$p" ]; then
    echo "== reference $p"
    "$here/_ref/$p" 2>&1 | grep -i -E "latency|avg|time|us" | head -12
  else
    echo "== reference $p: not built (make -C baseline)"
  fi
done
bin="$here/../topk_attn_b200/bin/ra_verify"
for m in center topk s1 s3; do
  echo "== ra_verify $m"
  "$bin" $m 2>&1 | grep -i -E "latency|us" | head -6
done
