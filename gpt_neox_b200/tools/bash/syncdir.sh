#!/usr/bin/env bash
# rsync a directory to the same path on every host of the hostfile.  usage: syncdir.sh <dir> [hostfile]
DIR=$(realpath "$1"); HOSTFILE=${2:-/job/hostfile}
for h in $(awk '{print $1}' "$HOSTFILE"); do rsync -az "$DIR/" "$h:$DIR/" & done; wait
