#!/bin/bash
# Tokenise a large jsonl corpus on several nodes at once: the input is split into one chunk per host of the hostfile,
# every host preprocesses its chunk with preprocess_data, and the pieces are merged into one indexed dataset.
#
#   multinode_prepare_data.sh <input.jsonl> <output-prefix> <hostfile> [extra preprocess_data args...]
#
# Needs pdsh and a shared filesystem (same assumptions as the cluster scripts under tools/bash).
set -euo pipefail
INPUT=$1; OUT=$2; HOSTFILE=$3; shift 3
HOSTS=$(awk '{print $1}' "$HOSTFILE" | paste -sd, -)
N=$(awk 'END{print NR}' "$HOSTFILE")
WORK=$(dirname "$OUT")/.prep_$$
mkdir -p "$WORK"
split -n l/"$N" -d --additional-suffix=.jsonl "$INPUT" "$WORK/chunk_"
i=0
for h in $(awk '{print $1}' "$HOSTFILE"); do
  f=$(printf "%s/chunk_%02d.jsonl" "$WORK" "$i")
  pdsh -w "$h" "cd $(pwd) && python -m gpt_neox_b200.tools.datasets.preprocess_data --input $f --output-prefix $WORK/part_$i $*" &
  i=$((i + 1))
done
wait
python -m gpt_neox_b200.tools.datasets.merge_datasets --input "$WORK" --output-prefix "$OUT"
echo "merged $N parts into $OUT (hosts: $HOSTS)"
