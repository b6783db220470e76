#!/usr/bin/env bash
# Stop every python process of the current user on all hosts of the hostfile (default /job/hostfile).
# Broader than kill.sh (which only targets train.py): meant for an operator cleaning up a wedged multi-node job
# from a cluster shell; the framework never calls it.
HOSTFILE=${1:-/job/hostfile}
pdsh -f 1024 -R ssh -w "$(awk '{print $1}' "$HOSTFILE" | paste -sd, -)" 'pkill -u "$USER" python'
