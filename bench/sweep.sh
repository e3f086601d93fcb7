#!/usr/bin/env bash
# The full AllReduce comparison on one 8-GPU box:
# this library (bin/allreduce), the unmodified reference programs (baseline/_ref)
# and stock NCCL (bench/backend_allreduce.py).  CSVs and a summary land in $OUT.
#
#   bench/sweep.sh [out_dir]        # needs: python -m stragglar_b200.build ; baseline/build_reference.sh <reference checkout>
set -u
cd "$(dirname "$0")/.."
OUT=${1:-sweep_out}; mkdir -p "$OUT"
SZ=1048576,16777216,67108864,268435456,1073741824
W=${STRAGGLAR_WARMUP:-10}; IT=${ITERS:-50}
run() { name=$1; shift; env "$@" STRAGGLAR_WARMUP=$W bin/allreduce $SIZES $ALGS $IT $DELAYS > "$OUT/$name.csv" 2> "$OUT/$name.err"; echo "$name: exit $?, $(grep -c VERIFY "$OUT/$name.err") verification failures"; }

# 8 GPUs: every algorithm, fp32 and bf16, straggler = last rank and physical rank 2
SIZES=$SZ ALGS=stragglar,stragglar_a2a,ring,rhd,direct,rsag DELAYS=-1,0,1,5,10 run ours_n8_fp32 X=1
SIZES=$SZ ALGS=stragglar,stragglar_a2a,ring,rhd,direct DELAYS=-1,0,1,5,10 run ours_n8_bf16 STRAGGLAR_DTYPE=bf16
SIZES=$SZ ALGS=stragglar,stragglar_a2a DELAYS=-1,5 run ours_n8_straggler2 STRAGGLAR_STRAGGLER=2
# 4 GPUs and the non-power-of-two 6-GPU schedule
SIZES=$SZ ALGS=stragglar,stragglar_a2a,ring,rhd,direct DELAYS=-1,0,1,5,10 run ours_n4 STRAGGLAR_NGPUS=4
SIZES=16777216,268435456,1073741824 ALGS=stragglar,stragglar_a2a,ring,direct DELAYS=5 run ours_n6 STRAGGLAR_NGPUS=6
STRAGGLAR_WARMUP=$W bin/reducescatter 1073741824 $IT > "$OUT/ours_reducescatter.csv" 2> "$OUT/ours_reducescatter.err"
# optional: buffers bound to NVLink multicast objects, in-switch reduction and replication (SWEEP_NVLS=1)
if [ "${SWEEP_NVLS:-0}" = 1 ]; then
  SIZES=$SZ ALGS=rsag,stragglar_a2a,stragglar DELAYS=-1,0,5 run ours_n8_nvls STRAGGLAR_NVLS=1
  SIZES=$SZ ALGS=rsag,stragglar_a2a,stragglar DELAYS=-1,0,5 run ours_n8_nvls_simta STRAGGLAR_NVLS=1 STRAGGLAR_PATH=simta
  STRAGGLAR_NVLS=1 STRAGGLAR_WARMUP=$W bin/reducescatter 1073741824 $IT > "$OUT/ours_reducescatter_nvls.csv" 2> "$OUT/ours_reducescatter_nvls.err"
fi

# the reference's programs (sizes padded as its pad_buffers.py prescribes for 8 GPUs)
if [ -x baseline/_ref/allreduce8 ]; then
  for s in 1053696 16780288 67113984 268441600 1073744896; do for a in stragglar ring rhd direct; do for d in -1 0 1 5 10; do
    baseline/_ref/allreduce8 $s $a $IT $d
  done; done; done > "$OUT/ref_n8.csv" 2> "$OUT/ref_n8.err"
  baseline/_ref/reducescatter 1073744896 $IT > "$OUT/ref_reducescatter.csv" 2>> "$OUT/ref_n8.err"
fi

# stock NCCL, 8 and 6 ranks
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29601 \
  bench/backend_allreduce.py --sizes $SZ --delays=-1,1,5,10 --iters $IT --warmup $W > "$OUT/nccl_n8.csv" 2> "$OUT/nccl_n8.err"
python -m torch.distributed.run --nnodes=1 --nproc-per-node 6 --master-addr 127.0.0.1 --master-port 29602 \
  bench/backend_allreduce.py --sizes 16777216,268435456,1073741824 --delays=5 --iters $IT --warmup $W > "$OUT/nccl_n6.csv" 2> "$OUT/nccl_n6.err"
python -m torch.distributed.run --nnodes=1 --nproc-per-node 6 --master-addr 127.0.0.1 --master-port 29603 \
  bench/sendrecv_allreduce.py --alg stragglar --sizes 16777216,268435456,1073741824 --delays=5 --iters 10 --warmup 3 > "$OUT/sendrecv_n6.csv" 2> "$OUT/sendrecv_n6.err"

python bench/summarize.py "$OUT"/ours_*.csv "$OUT"/ref_*.csv "$OUT"/nccl_*.csv "$OUT"/sendrecv_*.csv > "$OUT/summary.txt" 2>/dev/null
echo "summary: $OUT/summary.txt"
