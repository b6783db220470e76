#!/usr/bin/env bash
# Copy one file to the same path on every host of the hostfile.  usage: sync.sh <file> [hostfile]
FILE=$(realpath "$1"); HOSTFILE=${2:-/job/hostfile}
for h in $(awk '{print $1}' "$HOSTFILE"); do scp "$FILE" "$h:$FILE" & done; wait
