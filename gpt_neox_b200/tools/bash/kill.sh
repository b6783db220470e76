#!/usr/bin/env bash
# Stop training workers on every host of the hostfile (default /job/hostfile): pdsh ... 'pkill -f train.py'.
# Intended for an operator's own cluster shell; never called by the framework itself.
HOSTFILE=${1:-/job/hostfile}
pdsh -f 1024 -R ssh -w "$(awk '{print $1}' "$HOSTFILE" | paste -sd, -)" 'pkill -f train.py'
