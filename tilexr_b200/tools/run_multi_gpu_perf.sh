#!/bin/bash
# Runs every multi-GPU measurement of this repository on N GPUs of one node and leaves the
# results under OUT: bench (this library and the NCCL baseline), the collective sweep, the
# tensor-parallel MLP fusions (bf16 and block-scaled fp8), the fused all-reduce and the MoonEP stages at the
# shapes of cases/perf.json that are written for N ranks.
#   usage: run_multi_gpu_perf.sh N OUT
set -u
if [ $# -lt 2 ]; then echo "usage: $0 N OUT" >&2; exit 2; fi
N=$1
OUT=$2
mkdir -p "$OUT"
RUN="python -m torch.distributed.run --nnodes=1 --nproc-per-node $N --master-addr 127.0.0.1"
export NCCL_DEBUG=${NCCL_DEBUG:-WARN}
timeout 300 $RUN --master-port 29601 bench.py --gpus $N --steps 20 --warmup 5 > "$OUT/bench_tilexr.json" 2> "$OUT/bench_tilexr.err"
timeout 300 $RUN --master-port 29602 bench.py --gpus $N --steps 20 --warmup 5 --impl nccl > "$OUT/bench_nccl.json" 2> "$OUT/bench_nccl.err"
timeout 300 $RUN --master-port 29603 bench.py --gpus $N --steps 20 --warmup 5 --tokens 128 --no-e2e > "$OUT/bench_decode_tilexr.json" 2> "$OUT/bench_decode_tilexr.err"
timeout 300 $RUN --master-port 29604 bench.py --gpus $N --steps 20 --warmup 5 --tokens 128 --no-e2e --impl nccl > "$OUT/bench_decode_nccl.json" 2> "$OUT/bench_decode_nccl.err"
for op in all_gather all_to_all; do
  timeout 600 $RUN --master-port 29605 -m tilexr_b200.tools.collective_perf --op $op --min-bytes 4096 --max-bytes 1073741824 \
      --step-factor 4 --iters 10 --warmup-iters 3 --baseline nccl --symmetric 1 --csv "$OUT/${op}_symmetric.csv" > "$OUT/${op}_symmetric.txt" 2>&1
  timeout 600 $RUN --master-port 29606 -m tilexr_b200.tools.collective_perf --op $op --min-bytes 4096 --max-bytes 268435456 \
      --step-factor 4 --iters 10 --warmup-iters 3 --baseline nccl --symmetric 0 --csv "$OUT/${op}_staged.csv" > "$OUT/${op}_staged.txt" 2>&1
done
for op in all_reduce reduce_scatter broadcast; do
  timeout 600 $RUN --master-port 29607 -m tilexr_b200.tools.collective_perf --op $op --min-bytes 8192 --max-bytes 268435456 \
      --step-factor 8 --iters 10 --warmup-iters 3 --baseline nccl --symmetric 0 --csv "$OUT/${op}.csv" > "$OUT/${op}.txt" 2>&1
done
timeout 300 $RUN --master-port 29608 -m tilexr_b200.tools.tp_mlp_perf --tokens 8192 > "$OUT/tp_mlp.json" 2> "$OUT/tp_mlp.err"
timeout 300 $RUN --master-port 29609 -m tilexr_b200.tools.ar_norm_perf --hidden 8192 --batches 1,4,16,64,256,1024,4096,16384 > "$OUT/ar_norm.jsonl" 2> "$OUT/ar_norm.err"
for mode in benchmark prefetch reduce-grad; do
  timeout 300 $RUN --master-port 29610 -m tilexr_b200.tools.moonep.launcher --mode $mode --cases perf --iters 20 --warmup 5 \
      --json "$OUT/moonep_$mode.json" --csv "$OUT/moonep_$mode.csv" > "$OUT/moonep_$mode.txt" 2> "$OUT/moonep_$mode.err"
done
VLLM_TILEXR_COLLECTIVES=1 timeout 120 $RUN --master-port 29611 -m tilexr_b200.tools.vllm_collectives_smoke --count 65536 > "$OUT/vllm_smoke.json" 2> "$OUT/vllm_smoke.err"
tail -n 3 "$OUT"/*.err | cut -c1-300
ls -la "$OUT"
