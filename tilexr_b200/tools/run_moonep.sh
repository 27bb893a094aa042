#!/bin/bash
# MoonEP harness from end to end on N GPUs of one node (reference: scripts/run_moonep.sh and tools/moonep/launcher.py):
# correctness against the torch + NCCL reference backend, the stage benchmark with per-rank samples, the standalone
# PrefetchWeight and ReduceGrad benchmarks, the operator sequence of a training step (model flow), the dispatch hot loop, and
# the cross-rank aggregation of the samples into P50 / P99 tables.  `launcher --mode correctness --dump DIR` also leaves both
# sides' stage tensors for tools.moonep.tensor_dump (offline comparison) and tools.moonep.flowcharts (a chart of the stages).
#   usage: run_moonep.sh N OUT [correctness-cases] [perf-cases]      (case files under tilexr_b200/tools/moonep/cases/)
# Several nodes: run it on each node with the same OUT on a shared file system (or copy OUT/samples together) and
# finish with   python -m tilexr_b200.tools.moonep.launcher --mode aggregate --samples OUT/samples --json OUT/aggregate.json
# Without a GPU:  run_moonep.sh N OUT smoke host   runs the correctness mode and the dispatch hot loop as gloo ranks on a host-memory communicator.
set -u
if [ $# -lt 2 ]; then echo "usage: $0 N OUT [correctness-cases] [perf-cases]" >&2; exit 2; fi
N=$1
OUT=$2
CORRECT=${3:-correctness}
PERF=${4:-perf}
mkdir -p "$OUT/samples"
RUN="python -m torch.distributed.run --nnodes=1 --nproc-per-node $N --master-addr 127.0.0.1"
rc=0
if [ "$PERF" = "host" ]; then
    timeout 900 $RUN --master-port 29621 -m tilexr_b200.tools.moonep.launcher --mode correctness --backend host --cases "$CORRECT" \
        --json "$OUT/correctness.json" > "$OUT/correctness.md" 2> "$OUT/correctness.err" || rc=1
    timeout 600 $RUN --master-port 29626 -m tilexr_b200.tools.moonep.dispatch_hot_loop --backend host --cases "$CORRECT" --iters 20 --check-every 1 \
        --json "$OUT/dispatch_hot_loop.json" > "$OUT/dispatch_hot_loop.txt" 2> "$OUT/dispatch_hot_loop.err" || rc=1
    tail -n 2 "$OUT"/correctness.err "$OUT"/dispatch_hot_loop.err | cut -c1-300
    exit $rc
fi
timeout 900 $RUN --master-port 29621 -m tilexr_b200.tools.moonep.launcher --mode correctness --cases "$CORRECT" \
    --json "$OUT/correctness.json" > "$OUT/correctness.md" 2> "$OUT/correctness.err" || rc=1
timeout 600 $RUN --master-port 29622 -m tilexr_b200.tools.moonep.launcher --mode benchmark --cases "$PERF" --iters 20 --warmup 5 --trace \
    --samples "$OUT/samples" --json "$OUT/benchmark.json" --csv "$OUT/benchmark.csv" > "$OUT/benchmark.md" 2> "$OUT/benchmark.err" || rc=1
timeout 300 $RUN --master-port 29623 -m tilexr_b200.tools.moonep.launcher --mode prefetch --cases "$PERF" --iters 20 --warmup 5 \
    --json "$OUT/prefetch.json" --csv "$OUT/prefetch.csv" > "$OUT/prefetch.md" 2> "$OUT/prefetch.err" || rc=1
timeout 300 $RUN --master-port 29624 -m tilexr_b200.tools.moonep.launcher --mode reduce-grad --cases "$PERF" --iters 20 --warmup 5 \
    --json "$OUT/reduce_grad.json" --csv "$OUT/reduce_grad.csv" > "$OUT/reduce_grad.md" 2> "$OUT/reduce_grad.err" || rc=1
timeout 600 $RUN --master-port 29625 -m tilexr_b200.tools.moonep.launcher --mode model-flow --cases "$PERF" --layers 5 --iters 5 --warmup 1 \
    --json "$OUT/model_flow.json" > "$OUT/model_flow.md" 2> "$OUT/model_flow.err" || rc=1
timeout 600 $RUN --master-port 29626 -m tilexr_b200.tools.moonep.dispatch_hot_loop --cases "$PERF" --iters 100 --check-every 10 \
    --json "$OUT/dispatch_hot_loop.json" > "$OUT/dispatch_hot_loop.txt" 2> "$OUT/dispatch_hot_loop.err" || rc=1
python -m tilexr_b200.tools.moonep.launcher --mode aggregate --samples "$OUT/samples" --json "$OUT/aggregate.json" > "$OUT/aggregate.txt" 2>&1 || rc=1
tail -n 2 "$OUT"/*.err | cut -c1-300
exit $rc
