#!/usr/bin/env bash
# The AllReduce comparison of one 8-GPU box: this library (bin/allreduce), the unmodified reference programs
# (baseline/_ref) and stock NCCL (bench/backend_allreduce.py).  CSVs and a summary land in $OUT.
#
#   bench/sweep.sh [out_dir]        # needs: python -m stragglar_b200.build ; baseline/build_reference.sh <reference checkout>
#
# PARTS (default "n8 n4 n6 ref nccl") selects what runs; ITERS / STRAGGLAR_WARMUP default to 50 / 10 for this
# library, REF_ITERS to 20 for the reference's programs and NCCL.  A 4-GPU box runs PARTS="n4 ref nccl".
set -u
cd "$(dirname "$0")/.."
OUT=${1:-sweep_out}; mkdir -p "$OUT"
PARTS=${PARTS:-"n8 n4 n6 ref nccl"}
NG=$(nvidia-smi -L | wc -l)
SZ=${SIZES_ALL:-1048576,4194304,16777216,67108864,268435456,1073741824}
W=${STRAGGLAR_WARMUP:-10}; IT=${ITERS:-50}; RIT=${REF_ITERS:-20}
R="python -m torch.distributed.run --nnodes=1 --master-addr 127.0.0.1"
run() { name=$1; shift; env "$@" STRAGGLAR_WARMUP=$W bin/allreduce $SIZES $ALGS $IT $DELAYS > "$OUT/$name.csv" 2> "$OUT/$name.err"; echo "$name: exit $?, $(grep -c VERIFY "$OUT/$name.err") verification failures"; }
has() { case " $PARTS " in *" $1 "*) return 0;; *) return 1;; esac; }

if has n8 && [ "$NG" -ge 8 ]; then
  # every algorithm, fp32 and bf16, straggler = last rank and physical rank 2
  SIZES=$SZ ALGS=stragglar,stragglar_a2a,ring,rhd,direct,rsag DELAYS=-1,0,1,5,10 run ours_n8_fp32 X=1
  SIZES=$SZ ALGS=stragglar,stragglar_a2a,ring,rhd,direct,rsag DELAYS=-1,0,1,5,10 run ours_n8_bf16 STRAGGLAR_DTYPE=bf16
  SIZES=$SZ ALGS=stragglar,stragglar_a2a DELAYS=-1,5 run ours_n8_straggler2 STRAGGLAR_STRAGGLER=2
  STRAGGLAR_WARMUP=$W bin/reducescatter 1073741824 $IT > "$OUT/ours_reducescatter.csv" 2> "$OUT/ours_reducescatter.err"
fi
if has n4 && [ "$NG" -ge 4 ]; then
  SIZES=$SZ ALGS=stragglar,stragglar_a2a,ring,rhd,direct,rsag DELAYS=-1,0,1,5,10 run ours_n4 STRAGGLAR_NGPUS=4
fi
if has n6 && [ "$NG" -ge 6 ]; then
  # the non-power-of-two 6-GPU schedule (BASELINE.json config 4)
  SIZES=16777216,268435456,1073741824 ALGS=stragglar,stragglar_a2a,ring,direct DELAYS=5 run ours_n6 STRAGGLAR_NGPUS=6
fi
if has ref; then
  # the reference's programs, sizes padded as its pad_buffers.py prescribes (python -m stragglar_b200.pad <n>)
  if [ "$NG" -ge 8 ] && [ -x baseline/_ref/allreduce8 ]; then
    for s in 1053696 16780288 67113984 268441600 1073744896; do for a in stragglar ring rhd direct; do for d in -1 0 1 5 10; do
      baseline/_ref/allreduce8 $s $a $RIT $d
    done; done; done > "$OUT/ref_n8.csv" 2> "$OUT/ref_n8.err"
    baseline/_ref/reducescatter 1073744896 $RIT > "$OUT/ref_reducescatter.csv" 2>> "$OUT/ref_n8.err"
  fi
  if [ "$NG" -ge 4 ] && [ -x baseline/_ref/allreduce4 ]; then
    for s in 1050624 16779264 67110912 268437504 1073743872; do for a in stragglar ring rhd direct; do for d in -1 0 1 5 10; do
      CUDA_VISIBLE_DEVICES=0,1,2,3 baseline/_ref/allreduce4 $s $a $RIT $d
    done; done; done > "$OUT/ref_n4.csv" 2> "$OUT/ref_n4.err"
  fi
fi
if has nccl; then
  for n in 8 6 4; do
    [ "$NG" -ge $n ] || continue
    $R --nproc-per-node $n --master-port $((29600 + n)) bench/backend_allreduce.py --sizes $SZ --delays=-1,1,5,10 \
      --iters $RIT --warmup $W > "$OUT/nccl_n$n.csv" 2> "$OUT/nccl_n$n.err"
  done
  [ "$NG" -ge 8 ] && $R --nproc-per-node 8 --master-port 29618 bench/backend_allreduce.py --sizes $SZ --dtype bfloat16 --delays=-1,5 \
      --iters $RIT --warmup $W > "$OUT/nccl_n8_bf16.csv" 2> "$OUT/nccl_n8_bf16.err"
  # the library's n = 6 table executed the reference's way (grouped NCCL send/recv per round + separate adds)
  [ "$NG" -ge 6 ] && $R --nproc-per-node 6 --master-port 29603 bench/sendrecv_allreduce.py --alg stragglar \
      --sizes 16777216,268435456,1073741824 --delays=5 --iters 10 --warmup 3 > "$OUT/sendrecv_n6.csv" 2> "$OUT/sendrecv_n6.err"
fi
python bench/summarize.py "$OUT"/*.csv > "$OUT/summary.txt" 2>/dev/null
echo "summary: $OUT/summary.txt"
