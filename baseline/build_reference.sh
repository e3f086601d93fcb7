#!/usr/bin/env bash
# Builds the unmodified reference programs into baseline/_ref/ (git-ignored),
# with the command line of the reference README (README.md:26-30) plus an
# explicit Blackwell target, against the system NCCL:
#   baseline/_ref/allreduce4      <- stragglar/allreduce_4GPU.cu
#   baseline/_ref/allreduce8      <- stragglar/allreduce_8GPU.cu
#   baseline/_ref/reducescatter   <- stragglar/reducescatter.cu
# The reference's c10d backend (implementation/custom_backend) installs with
#   pip install --no-index --no-build-isolation --no-deps --target baseline/_ref <copy of custom_backend>
set -euo pipefail
REF=${1:?usage: build_reference.sh <path to a checkout of arjundevraj/stragglar>}
OUT="$(cd "$(dirname "$0")" && pwd)/_ref"
mkdir -p "$OUT"
ARCH="-gencode arch=compute_100,code=sm_100"
for pair in allreduce_4GPU:allreduce4 allreduce_8GPU:allreduce8 reducescatter:reducescatter; do
  src=${pair%%:*}; exe=${pair##*:}
  nvcc -diag-suppress=177 $ARCH -O2 -std=c++17 -o "$OUT/$exe" "$REF/stragglar/$src.cu" -lnccl
  echo "built $OUT/$exe"
done
